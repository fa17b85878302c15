// Block-select decode attention: FP16 old K + q4 old V + FP16 recent ring (and the
// dense-FP16-backed form of the same selection).
//
// Reference algorithm (cuda/kernels.cu:2832-3096), per q head:
//   score_b = (sum_{t in block b} q.K_t / len_b) / sqrt(hd) for every old block,
//   keep the top_n by score (ties -> lower block index, NaN / <= -1e30 never kept),
//   softmax-attend the tokens of the kept blocks plus the recent window.
// Here this is three launches:
//   1. block scores: one pass over old K per KV head (not per q head), using
//      sum_t q.K_t = q.(sum_t K_t): the kernel adds K rows (1 add per element) and takes
//      G dot products per block, so the scoring pass stays HBM-bound;
//   2. top-k per q head (iterative arg-max over the scores in shared memory);
//   3. attention over the selected tokens, split over CTAs, q4 V dequantised in registers
//      (value = f16(nibble * scale), kernels.cu:3085-3086), then the merge kernel.
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "attention.cuh"
#include "common.cuh"
#include "tc_ptx.cuh"

namespace {

struct SelArgs {
    const __half* old_k;     // head-major [slot][kvh][max_seq][hd] (compressed: old region; dense: K)
    const __half* ring_k;    // compressed: [slot][kvh][R][hd]; dense: null
    const __half* ring_v;
    const __half* dense_v;   // dense mode: V; compressed: null
    const uint8_t* q4_v;     // [slot][kvh][max_seq][hd/2]
    const float* q4_scale;   // [slot][kvh][max_seq]
    const float* q;          // [q_heads][hd]
    float* scores;           // [q_heads][score_stride]
    uint32_t* sel_blocks;    // [q_heads][64]
    float* sel_scores;       // [q_heads][64]
    float* part_m;
    float* part_l;
    float* part_o;
    uint32_t seq_id, max_seq_len, kv_heads, q_heads, hd;
    uint32_t seq_len, old_len, recent_window, ring_size, block_size, nb, top_n;
    uint32_t block_begin, block_end;  // blocks this call may read (split-K); [0, nb) otherwise
    uint32_t score_stride, include_recent, splits;
    float inv_sqrt;
    uint32_t* status_word;  // the context's device status word
};

// ---- 1. block scores. grid (ceil(blocks/4), kv_heads), 128 threads; a warp per block. ----
template <int HD>
__global__ void __launch_bounds__(128) block_score_kernel(SelArgs a) {
    constexpr int LPT = HD / 8;        // lanes per token row (16-byte pieces)
    constexpr int TPI = 32 / LPT;      // tokens per warp-wide load
    extern __shared__ float sq[];      // q of this kv head's group: [G][HD]
    pdl_wait();
    pdl_trigger();
    const uint32_t kvh = blockIdx.y;
    const uint32_t G = a.q_heads / a.kv_heads;
    for (uint32_t i = threadIdx.x; i < G * HD; i += blockDim.x) sq[i] = a.q[(size_t)kvh * G * HD + i];
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t b = a.block_begin + blockIdx.x * 4u + warp;
    if (b >= a.block_end) return;
    const uint32_t t0 = b * a.block_size;
    const uint32_t t1 = min(t0 + a.block_size, a.old_len);
    const __half* Kh = a.old_k + kv_row_offset(a.seq_id, kvh, 0, a.kv_heads, a.max_seq_len, HD);
    const uint32_t sub = lane / LPT, piece = lane % LPT;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll 8
    for (uint32_t t = t0 + sub; t < t1; t += TPI) {
        const uint4 w = *reinterpret_cast<const uint4*>(Kh + (size_t)t * HD + piece * 8);
        const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
        }
    }
    // fold the token sub-groups together: lanes with equal `piece` hold the same dims
#pragma unroll
    for (int o = 16; o >= LPT; o >>= 1)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    const float inv_len = 1.0f / (float)(t1 - t0);
    for (uint32_t g = 0; g < G; ++g) {
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) dot = fmaf(sq[g * HD + piece * 8 + j], acc[j], dot);
        // reduce over the LPT lanes that hold distinct pieces
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) a.scores[(size_t)(kvh * G + g) * a.score_stride + (b - a.block_begin)] = (dot * inv_len) * a.inv_sqrt;
    }
}

// ---- 1b. block scores with the K rows staged by bulk copies. Same grid and result as block_score_kernel; the CTA's
// four blocks (contiguous in the head-major cache) arrive as four 1-D bulk async copies on one mbarrier, so all of a
// launch's bytes are in flight at once and the pass costs one memory round trip plus the transfer instead of a chain
// of dependent loads per warp. Shared memory: q of the group [G][HD] f32, then 4 x block_size x HD f16.
template <int HD>
__global__ void __launch_bounds__(128) block_score_bulk_kernel(SelArgs a) {
    constexpr int DPL = HD / 32;  // dims per lane
    extern __shared__ __align__(128) unsigned char bs_smem[];
    __shared__ uint64_t bar;
    const uint32_t G = a.q_heads / a.kv_heads;
    float* sq = reinterpret_cast<float*>(bs_smem);
    __half* sk = reinterpret_cast<__half*>(bs_smem + (((size_t)G * HD * sizeof(float) + 127u) & ~(size_t)127u));
    const uint32_t kvh = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t b_first = a.block_begin + blockIdx.x * 4u;
    const __half* Kh = a.old_k + kv_row_offset(a.seq_id, kvh, 0, a.kv_heads, a.max_seq_len, HD);
    // q, and the newest old K row (an append evicts the ring's oldest token into the old region), come from the
    // kernel before this one
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        uint32_t total = 0;
        for (uint32_t w = 0; w < 4u; ++w) {
            const uint32_t b = b_first + w;
            if (b >= a.block_end) break;
            const uint32_t t0 = b * a.block_size, t1 = min(t0 + a.block_size, a.old_len);
            total += (t1 - t0) * HD * 2u;
        }
        tc::mbar_expect_tx(&bar, total);
        for (uint32_t w = 0; w < 4u; ++w) {
            const uint32_t b = b_first + w;
            if (b >= a.block_end) break;
            const uint32_t t0 = b * a.block_size, t1 = min(t0 + a.block_size, a.old_len);
            const uint32_t bytes = (t1 - t0) * HD * 2u;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(tc::smem_u32(sk + (size_t)w * a.block_size * HD)), "l"(Kh + (size_t)t0 * HD), "r"(bytes),
                           "r"(tc::smem_u32(&bar)) : "memory");
        }
    }
    for (uint32_t i = threadIdx.x; i < G * HD; i += blockDim.x) sq[i] = a.q[(size_t)kvh * G * HD + i];
    __syncthreads();  // also publishes the barrier's initialisation
    const bool landed = tc::mbar_wait(&bar, 0u);
    if (!landed) {  // never seen; the copies may still be in flight, so the CTA may not leave its shared memory yet
        if (threadIdx.x == 0) atomicOr(a.status_word, 4u);
        tc::mbar_wait(&bar, 0u);
        return;
    }
    const uint32_t b = b_first + warp;
    if (b >= a.block_end) return;
    const uint32_t t0 = b * a.block_size, t1 = min(t0 + a.block_size, a.old_len), n = t1 - t0;
    const __half* rows = sk + (size_t)warp * a.block_size * HD + lane * DPL;
    float acc[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[j] = 0.0f;
#pragma unroll 8
    for (uint32_t t = 0; t < n; ++t) {
        if (DPL == 4) {
            const uint2 w = *reinterpret_cast<const uint2*>(rows + (size_t)t * HD);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
            acc[0] += f0.x, acc[1] += f0.y, acc[DPL - 2] += f1.x, acc[DPL - 1] += f1.y;
        } else {
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(rows + (size_t)t * HD));
            acc[0] += f0.x, acc[1] += f0.y;
        }
    }
    const float inv_len = 1.0f / (float)n;
    for (uint32_t g = 0; g < G; ++g) {
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) dot = fmaf(sq[g * HD + lane * DPL + j], acc[j], dot);
        dot = warp_sum(dot);
        if (lane == 0) a.scores[(size_t)(kvh * G + g) * a.score_stride + (b - a.block_begin)] = (dot * inv_len) * a.inv_sqrt;
    }
}

// ---- 2a. top-k by rank, for up to 4096 candidates per q head. A candidate's place in the descending list is the
// number of selectable candidates that beat it (greater score, or equal score and lower block index), which is exactly
// the order the iterative arg-max below produces, so the whole selection is one pass. Scores that are NaN or <= -1e30
// are never selectable. The candidates of a head are cut into `slices` (gridDim.y) so that the ranking spreads over
// the whole GPU instead of one CTA per head: CTA (h, s) ranks its slice against all candidates held in shared memory
// and writes the winners among them; list positions past the number of selectable candidates are filled as empty.
//
// Candidate c of head h: score at scores[h * head_stride + (c / per_part) * part_stride + (c % per_part) * elem_stride],
// block index = ids[same offset] when `ids` is given (gathered (score, index) pairs), else index_base + c.
struct RankArgs {
    const float* scores;
    const uint32_t* ids;
    uint32_t* out_ids;     // [q_heads][64 * out_stride], element (h, r) at (h * 64 + r) * out_stride
    float* out_scores;     // same addressing
    size_t head_stride, part_stride;
    uint32_t per_part, elem_stride, n, index_base, top_n, out_stride;
};

__global__ void __launch_bounds__(256) rank_topk_kernel(RankArgs a) {
    extern __shared__ __align__(16) float rk_smem[];
    const uint32_t n4 = (a.n + 3u) / 4u;                      // candidates padded to whole groups of four
    float* sc = rk_smem;                                      // 4 n4 scores, unselectable ones replaced by -inf
    uint32_t* id = reinterpret_cast<uint32_t*>(sc + 4u * n4); // 4 n4 block indices
    __shared__ uint32_t s_selectable;
    pdl_wait();
    pdl_trigger();
    const uint32_t h = blockIdx.x, slice = blockIdx.y, slices = gridDim.y, tid = threadIdx.x;
    if (tid == 0) s_selectable = 0;
    __syncthreads();
    uint32_t mine = 0;
    for (uint32_t c = tid; c < 4u * n4; c += blockDim.x) {
        float s = -INFINITY;
        uint32_t b = 0xffffffffu;
        if (c < a.n) {
            const size_t off = (size_t)h * a.head_stride + (size_t)(c / a.per_part) * a.part_stride +
                               (size_t)(c % a.per_part) * a.elem_stride;
            s = a.scores[off];
            b = a.ids ? a.ids[off] : a.index_base + c;
        }
        const bool ok = s > -1e30f && b != 0xffffffffu;  // false for NaN too
        sc[c] = ok ? s : -INFINITY;
        id[c] = b;
        mine += ok ? 1u : 0u;
    }
    mine = (uint32_t)__reduce_add_sync(0xffffffffu, mine);
    if ((tid & 31u) == 0u && mine) atomicAdd(&s_selectable, mine);
    __syncthreads();
    const uint32_t filled = min(s_selectable, a.top_n);  // list positions that will receive a winner
    // empty tail of the list, dealt to the slices
    for (uint32_t r = filled + slice * blockDim.x + tid; r < 64u; r += slices * blockDim.x) {
        a.out_ids[((size_t)h * 64u + r) * a.out_stride] = 0xffffffffu;
        a.out_scores[((size_t)h * 64u + r) * a.out_stride] = -1e30f;
    }
    // four adjacent lanes share one candidate of this slice; lane `part` scans the groups of four part, part + 4, ...
    // (16-byte shared-memory reads, four independent counters)
    const uint32_t per_slice = (a.n + slices - 1u) / slices;
    const uint32_t c0 = slice * per_slice, c1 = min(c0 + per_slice, a.n);
    const uint32_t part = tid & 3u;
    const float4* sc4 = reinterpret_cast<const float4*>(sc);
    const uint4* id4 = reinterpret_cast<const uint4*>(id);
    for (uint32_t i0 = c0; i0 < c1; i0 += blockDim.x / 4u) {
        const uint32_t i = i0 + tid / 4u;
        const float s = i < c1 ? sc[i] : -INFINITY;
        const uint32_t bi = i < c1 ? id[i] : 0u;
        uint32_t r0 = 0, r1 = 0, r2 = 0, r3 = 0;
        if (s != -INFINITY) {
#pragma unroll 4
            for (uint32_t j = part; j < n4; j += 4u) {
                const float4 o = sc4[j];
                const uint4 b = id4[j];
                // equal score, lower block index: ahead
                r0 += (o.x > s || (o.x == s && b.x < bi)) ? 1u : 0u;
                r1 += (o.y > s || (o.y == s && b.y < bi)) ? 1u : 0u;
                r2 += (o.z > s || (o.z == s && b.z < bi)) ? 1u : 0u;
                r3 += (o.w > s || (o.w == s && b.w < bi)) ? 1u : 0u;
            }
        }
        uint32_t rank = (r0 + r1) + (r2 + r3);
        rank += __shfl_xor_sync(0xffffffffu, rank, 1);
        rank += __shfl_xor_sync(0xffffffffu, rank, 2);
        if (part == 0 && s != -INFINITY && rank < a.top_n && rank < 64u) {
            a.out_ids[((size_t)h * 64u + rank) * a.out_stride] = bi;
            a.out_scores[((size_t)h * 64u + rank) * a.out_stride] = s;
        }
    }
}

// ---- 2. top-k. grid q_heads, 128 threads. scores -> sel_blocks/sel_scores (descending). ----
__global__ void __launch_bounds__(128) topk_blocks_kernel(SelArgs a) {
    extern __shared__ float sc[];  // nb scores
    __shared__ float wbest[4];
    __shared__ uint32_t wbidx[4];
    const uint32_t h = blockIdx.x;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    for (uint32_t i = threadIdx.x; i < a.nb; i += blockDim.x) sc[i] = a.scores[(size_t)h * a.score_stride + i];
    for (uint32_t i = threadIdx.x; i < 64u; i += blockDim.x) {
        a.sel_blocks[h * 64u + i] = 0xffffffffu;
        a.sel_scores[h * 64u + i] = -1e30f;
    }
    __syncthreads();
    for (uint32_t k = 0; k < a.top_n; ++k) {
        // a candidate must compare greater than -1e30 (the reference's empty-slot score); NaN never does
        float best = -1e30f;
        uint32_t bidx = 0xffffffffu;
        for (uint32_t i = threadIdx.x; i < a.nb; i += blockDim.x) {
            const float s = sc[i];
            if (s > best) {  // strided scan keeps the lowest index among equal scores per thread
                best = s;
                bidx = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bidx, o);
            if (ob > best || (ob == best && oi < bidx)) {
                best = ob;
                bidx = oi;
            }
        }
        if (lane == 0) {
            wbest[warp] = best;
            wbidx[warp] = bidx;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float fb = wbest[0];
            uint32_t fi = wbidx[0];
            for (int w = 1; w < 4; ++w)
                if (wbest[w] > fb || (wbest[w] == fb && wbidx[w] < fi)) {
                    fb = wbest[w];
                    fi = wbidx[w];
                }
            if (fi != 0xffffffffu) {
                a.sel_blocks[h * 64u + k] = fi;
                a.sel_scores[h * 64u + k] = fb;
                sc[fi] = -INFINITY;  // never compares greater than -1e30 again
            }
            wbidx[0] = fi;
        }
        __syncthreads();
        if (wbidx[0] == 0xffffffffu) break;  // nothing selectable is left
        __syncthreads();
    }
}

// ---- 3. attention over the selected tokens. grid (splits, q_heads), 128 threads. ----
// Slot space: [0, 64*block_size) = selected blocks in list order (empty entries and tokens past
// old_len are skipped), then the recent tokens [old_len, seq_len). DENSE: K/V from the dense cache.
template <int HD, bool DENSE>
__global__ void __launch_bounds__(128) selected_attend_kernel(SelArgs a) {
    constexpr int DPL = HD / 32;  // dims per lane (4 for 128, 2 for 64), contiguous
    __shared__ uint32_t sblk[64];
    __shared__ float sm_m[4], sm_l[4], sm_o[4][HD];
    pdl_wait();
    pdl_trigger();
    const uint32_t split = blockIdx.x, h = blockIdx.y;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t G = a.q_heads / a.kv_heads, kvh = h / G;
    if (threadIdx.x < 64) {
        uint32_t b = a.sel_blocks[h * 64u + threadIdx.x];
        if (b != 0xffffffffu && (b < a.block_begin || b >= a.block_end)) b = 0xffffffffu;
        sblk[threadIdx.x] = b;
    }
    __syncthreads();
    const uint32_t sel_slots = 64u * a.block_size;
    const uint32_t recent_n = a.include_recent ? a.seq_len - a.old_len : 0u;
    const uint32_t total = sel_slots + recent_n;
    uint32_t per = (total + a.splits - 1) / a.splits;
    per = (per + 3u) & ~3u;
    const uint32_t s0 = min(split * per, total), s1 = min(s0 + per, total);
    const size_t head_base = kv_row_offset(a.seq_id, kvh, 0, a.kv_heads, a.max_seq_len, HD);
    const size_t vec_base = ((size_t)a.seq_id * a.kv_heads + kvh) * (size_t)a.max_seq_len;
    const size_t ring_base = DENSE ? 0 : kv_row_offset(a.seq_id, kvh, 0, a.kv_heads, a.ring_size, HD);
    float qr[DPL], acc[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
        qr[j] = a.q[(size_t)h * HD + lane * DPL + j];
        acc[j] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    // A warp takes U consecutive slots per pass and issues every load of the pass (K rows, then V rows / q4 bytes
    // and scales) before it uses any of them: the pass costs one memory latency instead of U.
    constexpr int U = 8;
    for (uint32_t base = s0 + warp * U; base < s1; base += 4u * U) {
        uint32_t tok[U];
        bool live[U], old_tok[U];
        {
            // one division pair per pass: the U slots are consecutive, so list position, offset in the block and
            // ring position are carried
            uint32_t li = 0, off = 0, rpos = 0, rt = 0;
            if (base < sel_slots) li = base / a.block_size, off = base % a.block_size;
            const uint32_t first_recent = base < sel_slots ? sel_slots : base;  // first slot of the pass in the ring part
            rt = a.old_len + (first_recent - sel_slots);
            if (!DENSE && a.ring_size) rpos = rt % a.ring_size;
#pragma unroll
            for (int i = 0; i < U; ++i) {
                const uint32_t slot = base + i;
                live[i] = slot < s1;
                old_tok[i] = false;
                tok[i] = 0;
                if (slot < sel_slots) {
                    const uint32_t b = sblk[li < 64u ? li : 63u];
                    const uint32_t t = b * a.block_size + off;
                    if (b == 0xffffffffu || t >= a.old_len) live[i] = false;
                    else tok[i] = t, old_tok[i] = true;
                    if (++off == a.block_size) off = 0, ++li;
                } else {
                    // dense form: the token index; ring form: the ring row of that token
                    tok[i] = DENSE ? rt : rpos;
                    ++rt;
                    if (++rpos == a.ring_size) rpos = 0;
                }
            }
        }
        uint2 kw[U], vw[U];
        float vscale[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
            kw[i] = make_uint2(0u, 0u);
            if (!live[i]) continue;
            const __half* kp = (DENSE || old_tok[i]) ? a.old_k + head_base + (size_t)tok[i] * HD
                                                     : a.ring_k + ring_base + (size_t)tok[i] * HD;
            if (DPL == 4) kw[i] = *reinterpret_cast<const uint2*>(kp + lane * 4);
            else kw[i].x = *reinterpret_cast<const uint32_t*>(kp + lane * 2);
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
            vw[i] = make_uint2(0u, 0u);
            vscale[i] = 0.0f;
            if (!live[i]) continue;
            if (!DENSE && old_tok[i]) {
                vscale[i] = a.q4_scale[vec_base + tok[i]];
                const uint8_t* vp = a.q4_v + (vec_base + tok[i]) * (HD / 2) + lane * (DPL / 2);
                if (DPL == 4) vw[i].x = *reinterpret_cast<const uint16_t*>(vp);
                else vw[i].x = *vp;
            } else {
                const __half* vp = DENSE ? a.dense_v + head_base + (size_t)tok[i] * HD
                                         : a.ring_v + ring_base + (size_t)tok[i] * HD;
                if (DPL == 4) vw[i] = *reinterpret_cast<const uint2*>(vp + lane * 4);
                else vw[i].x = *reinterpret_cast<const uint32_t*>(vp + lane * 2);
            }
        }
        float sc[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&kw[i].x));
            float dot = fmaf(qr[0], f0.x, 0.0f);
            dot = fmaf(qr[1], f0.y, dot);
            if (DPL == 4) {
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&kw[i].y));
                dot = fmaf(qr[DPL - 2], f1.x, dot);
                dot = fmaf(qr[DPL - 1], f1.y, dot);
            }
            sc[i] = dot;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < U; ++i) sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], o);
#pragma unroll
        for (int i = 0; i < U; ++i) {
            if (!live[i]) continue;  // warp-uniform
            const float s = sc[i] * a.inv_sqrt;
            float vx[DPL];
            if (!DENSE && old_tok[i]) {
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    // signed nibble as an exact float without a conversion instruction: 2^23 + (nib ^ 8) - (2^23 + 8)
                    const uint32_t nib = (vw[i].x >> (4 * j)) & 0xfu;
                    const float sv = __uint_as_float(0x4B000000u | (nib ^ 8u)) - 8388616.0f;
                    vx[j] = __half2float(__float2half_rn(sv * vscale[i]));
                }
            } else {
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&vw[i].x));
                vx[0] = f0.x; vx[1] = f0.y;
                if (DPL == 4) {
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&vw[i].y));
                    vx[DPL - 2] = f1.x; vx[DPL - 1] = f1.y;
                }
            }
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn);
            const float pw = expf(s - mn);
            l = l * corr + pw;
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[j] = fmaf(pw, vx[j], acc[j] * corr);
            m = mn;
        }
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int j = 0; j < DPL; ++j) sm_o[warp][lane * DPL + j] = acc[j];
    __syncthreads();
    for (uint32_t d = threadIdx.x; d < HD; d += blockDim.x) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float e = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - M);
            L += sm_l[w] * e;
            O += sm_o[w][d] * e;
        }
        const size_t pi = (size_t)h * a.splits + split;
        if (d == 0) {
            a.part_m[pi] = M;
            a.part_l[pi] = L;
        }
        a.part_o[pi * HD + d] = O;
    }
}

// ---- 3b. attention over the selected tokens with K and V staged by bulk copies (compressed cache only).
// Work items per q head: runs of up to 32 tokens of the 64 selected blocks (K f16 rows and q4 V rows of a block are
// contiguous in the head-major cache) followed by pieces of the recent ring (`ring_piece` slots each: K and V f16).
// A warp takes one item: two bulk async copies into its own slice of shared memory on its own mbarrier, so all of a
// launch's bytes are in flight at once, where the gather form issues them as dependent rounds of loads. The item's
// dot products are reduced across the warp by a halving exchange (31 shuffles for 32 sums, lane t ends up with token
// t's score), the softmax runs one token per lane, and only the V accumulation walks the tokens one by one. grid (ceil(items / warps), q_heads), `warps` x 32 threads; one (m, l, o) partial per CTA, merged
// by the same kernel as before.
constexpr uint32_t STAGED_MAX_WARPS = 16;
constexpr uint32_t STAGED_ITEM_TOKENS = 32;  // tokens per work item (one per lane in the softmax)

// v[i] (i < 32) is this lane's partial sum for token i. Returns the complete sum of token `lane`.
__device__ __forceinline__ float transpose_reduce32(float (&v)[32], uint32_t lane) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        const bool upper = (lane & o) != 0u;
#pragma unroll
        for (int i = 0; i < o; ++i) {
            // keep the half of the values that matches this lane's bit, hand the other half to the partner
            const float keep = upper ? v[i + o] : v[i];
            const float give = upper ? v[i] : v[i + o];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, give, o);
        }
    }
    return v[0];
}

template <int HD>
__global__ void __launch_bounds__(32 * STAGED_MAX_WARPS) selected_attend_staged_kernel(SelArgs a, uint32_t slice_bytes,
                                                                                       uint32_t ring_piece,
                                                                                       uint32_t ring_items) {
    constexpr int DPL = HD / 32;  // dims per lane, contiguous
    extern __shared__ __align__(128) unsigned char st_smem[];
    __shared__ uint64_t bars[STAGED_MAX_WARPS];
    __shared__ float sm_m[STAGED_MAX_WARPS], sm_l[STAGED_MAX_WARPS], sm_o[STAGED_MAX_WARPS][HD];
    const uint32_t h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    const uint32_t G = a.q_heads / a.kv_heads, kvh = h / G;
    const uint32_t item = blockIdx.x * warps + warp;
    unsigned char* slice = st_smem + (size_t)warp * slice_bytes;
    pdl_wait();
    pdl_trigger();
    // ---- what this warp's item is
    uint32_t n = 0, tok0 = 0;
    bool ring = false;
    const uint32_t subs = (a.block_size + STAGED_ITEM_TOKENS - 1u) / STAGED_ITEM_TOKENS;  // items per selected block
    if (item < 64u * subs) {
        const uint32_t b = a.sel_blocks[h * 64u + item / subs], off = (item % subs) * STAGED_ITEM_TOKENS;
        if (b != 0xffffffffu && b >= a.block_begin && b < a.block_end) {
            tok0 = b * a.block_size + off;
            if (tok0 < a.old_len) n = min(min(STAGED_ITEM_TOKENS, a.block_size - off), a.old_len - tok0);
        }
    } else if (a.include_recent && item - 64u * subs < ring_items) {
        ring = true;
        const uint32_t recent_n = a.seq_len - a.old_len;  // the ring's live slots are [0, recent_n)
        tok0 = (item - 64u * subs) * ring_piece;
        if (tok0 < recent_n) n = min(ring_piece, recent_n - tok0);
    }
    const size_t vec_base = ((size_t)a.seq_id * a.kv_heads + kvh) * (size_t)a.max_seq_len;
    const uint32_t k_bytes = n * HD * 2u, v_bytes = ring ? k_bytes : n * (HD / 2u);
    if (lane == 0 && n) {
        tc::mbar_init(&bars[warp], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::mbar_expect_tx(&bars[warp], k_bytes + v_bytes);
        const void *ksrc, *vsrc;
        if (ring) {
            const size_t off = kv_row_offset(a.seq_id, kvh, tok0, a.kv_heads, a.ring_size, HD);
            ksrc = a.ring_k + off;
            vsrc = a.ring_v + off;
        } else {
            ksrc = a.old_k + kv_row_offset(a.seq_id, kvh, tok0, a.kv_heads, a.max_seq_len, HD);
            vsrc = a.q4_v + (vec_base + tok0) * (HD / 2u);
        }
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(tc::smem_u32(slice)), "l"(ksrc), "r"(k_bytes), "r"(tc::smem_u32(&bars[warp])) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(tc::smem_u32(slice + k_bytes)), "l"(vsrc), "r"(v_bytes), "r"(tc::smem_u32(&bars[warp])) : "memory");
    }
    float qr[DPL], acc[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
        qr[j] = a.q[(size_t)h * HD + lane * DPL + j] * a.inv_sqrt;
        acc[j] = 0.0f;
    }
    // the q4 scale of this lane's token (old blocks only), requested before the wait
    float scale = 0.0f;
    if (!ring && lane < n) scale = a.q4_scale[vec_base + tok0 + lane];
    float m = -INFINITY, l = 0.0f;
    __syncwarp();
    if (n) {
        if (!tc::mbar_wait(&bars[warp], 0u)) {  // never seen; wait on, the copies target this CTA's shared memory
            if (lane == 0) atomicOr(a.status_word, 4u);
            tc::mbar_wait(&bars[warp], 0u);
            n = 0;
        }
    }
    const __half* sK = reinterpret_cast<const __half*>(slice) + lane * DPL;
    const unsigned char* sV = slice + k_bytes;
    if (n) {
        const uint32_t g0 = 0, cnt = n;  // warp-uniform, at most 32
        // ---- 32 dot products, dims split over the lanes, then the halving exchange
        float part[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const uint32_t t = g0 + min((uint32_t)i, cnt - 1u);
            if (DPL == 4) {
                const uint2 w = *reinterpret_cast<const uint2*>(sK + (size_t)t * HD);
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
                part[i] = fmaf(qr[DPL - 1], f1.y, fmaf(qr[DPL - 2], f1.x, fmaf(qr[1], f0.y, qr[0] * f0.x)));
            } else {
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(sK + (size_t)t * HD));
                part[i] = fmaf(qr[1], f0.y, qr[0] * f0.x);
            }
        }
        float s = transpose_reduce32(part, lane);  // token g0 + lane (already scaled by 1/sqrt(hd) through q)
        if (lane >= cnt) s = -INFINITY;
        // ---- softmax, one token per lane
        const float mn = fmaxf(m, warp_max(s));
        const float corr = expf(m - mn);            // 0 on the first group (m = -inf, mn finite)
        const float p = lane < cnt ? expf(s - mn) : 0.0f;
        l = l * corr + warp_sum(p);
        m = mn;
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[j] *= corr;
        // ---- O += P V, token by token
#pragma unroll 4
        for (uint32_t i = 0; i < cnt; ++i) {
            const float pw = __shfl_sync(0xffffffffu, p, i);
            const uint32_t t = g0 + i;
            float vx[DPL];
            if (!ring) {
                const float sc = __shfl_sync(0xffffffffu, scale, i);
                uint32_t bits;
                if (DPL == 4) bits = *reinterpret_cast<const uint16_t*>(sV + (size_t)t * (HD / 2) + lane * 2);
                else bits = sV[(size_t)t * (HD / 2) + lane];
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    // signed nibble as an exact float without a conversion instruction: 2^23 + (nib ^ 8) - (2^23 + 8)
                    const uint32_t nib = (bits >> (4 * j)) & 0xfu;
                    const float sv = __uint_as_float(0x4B000000u | (nib ^ 8u)) - 8388616.0f;
                    vx[j] = __half2float(__float2half_rn(sv * sc));
                }
            } else {
                const __half* vp = reinterpret_cast<const __half*>(sV) + (size_t)t * HD + lane * DPL;
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(vp));
                vx[0] = f0.x, vx[1] = f0.y;
                if (DPL == 4) {
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(vp + 2));
                    vx[DPL - 2] = f1.x, vx[DPL - 1] = f1.y;
                }
            }
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[j] = fmaf(pw, vx[j], acc[j]);
        }
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int j = 0; j < DPL; ++j) sm_o[warp][lane * DPL + j] = acc[j];
    __syncthreads();
    for (uint32_t d = threadIdx.x; d < HD; d += blockDim.x) {
        float M = -INFINITY;
        for (uint32_t w = 0; w < warps; ++w) M = fmaxf(M, sm_m[w]);
        float L = 0.0f, O = 0.0f;
        for (uint32_t w = 0; w < warps; ++w) {
            const float e = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - M);
            L += sm_l[w] * e;
            O += sm_o[w][d] * e;
        }
        const size_t pi = (size_t)h * a.splits + blockIdx.x;
        if (d == 0) {
            a.part_m[pi] = M;
            a.part_l[pi] = L;
        }
        a.part_o[pi * HD + d] = O;
    }
}

// Shape of the staged attend launch for this call, or splits == 0 when the gather form has to be used.
struct StagedPlan {
    uint32_t slice_bytes, ring_piece, ring_items, warps, splits;
};

StagedPlan plan_staged(const SelArgs& a, bool dense, int sm_count) {
    StagedPlan p = {};
    if (dense || a.block_size == 0u) return p;
    const uint32_t item_tokens = a.block_size < STAGED_ITEM_TOKENS ? a.block_size : STAGED_ITEM_TOKENS;
    uint32_t slice = item_tokens * (a.hd * 2u + a.hd / 2u);
    slice = (slice + 127u) & ~127u;
    uint32_t piece = slice / (a.hd * 4u);  // ring slots whose K and V rows (f16) fit one slice
    if (piece > 8u) piece &= ~7u;
    if (piece == 0u) return p;
    const uint32_t recent_n = a.seq_len - a.old_len;
    p.slice_bytes = slice;
    p.ring_piece = piece;
    p.ring_items = (recent_n + piece - 1u) / piece;
    const uint32_t subs = (a.block_size + STAGED_ITEM_TOKENS - 1u) / STAGED_ITEM_TOKENS;
    if (subs > 64u) return p;
    const uint32_t items = 64u * subs + p.ring_items;
    // warps (= items) per CTA: the fewest for which the whole launch is resident at once; a second wave that holds
    // a handful of CTAs would double the time of this latency-bound kernel
    const uint32_t sms = sm_count > 0 ? (uint32_t)sm_count : 1u;
    p.warps = STAGED_MAX_WARPS;
    for (uint32_t w = 4u; w <= STAGED_MAX_WARPS; ++w) {
        uint32_t per_sm = (220u * 1024u) / (w * slice + 10u * 1024u);  // dynamic slices + the static merge arrays
        if (per_sm > 2048u / (32u * w)) per_sm = 2048u / (32u * w);
        const uint32_t ctas = a.q_heads * ((items + w - 1u) / w);
        if (per_sm >= 1u && ctas <= per_sm * sms) {
            p.warps = w;
            break;
        }
    }
    p.splits = (items + p.warps - 1u) / p.warps;
    if (p.splits > 256u) p.splits = 0;  // the merge kernel's limit
    return p;
}

struct SelPlan {
    uint32_t old_len, nb, top_n, recent_count;
};

int fill_common(const M40llmKVCache* kv, SelArgs* a, uint32_t seq_id, const void* q, uint32_t q_heads,
                uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, bool dense) {
    a->seq_id = seq_id;
    a->max_seq_len = kv->max_seq_len;
    a->kv_heads = kv->num_heads;
    a->q_heads = q_heads;
    a->hd = kv->head_dim;
    a->seq_len = seq_len;
    a->recent_window = recent_window;
    a->ring_size = dense ? 0u : kv->recent_window;
    a->block_size = block_size;
    a->old_len = seq_len > recent_window ? seq_len - recent_window : 0u;
    a->nb = a->old_len == 0 ? 0u : (a->old_len + block_size - 1) / block_size;
    a->top_n = top_blocks < a->nb ? top_blocks : a->nb;
    a->block_begin = 0;
    a->block_end = a->nb;
    a->score_stride = a->nb ? a->nb : 1u;
    a->include_recent = 1;
    a->inv_sqrt = attn_inv_sqrt(kv->head_dim);
    a->q = (const float*)q;
    if (dense) {
        a->old_k = kv->d_k;
        a->dense_v = kv->d_v;
        a->ring_k = a->ring_v = nullptr;
        a->q4_v = nullptr;
        a->q4_scale = nullptr;
    } else {
        a->old_k = kv->d_old_k;
        a->dense_v = nullptr;
        a->ring_k = kv->d_recent_k;
        a->ring_v = kv->d_recent_v;
        a->q4_v = kv->d_q4_v;
        a->q4_scale = kv->d_q4_scale;
    }
    return 0;
}

int launch_scores(M40llmCudaContext* ctx, const SelArgs& a0) {
    const uint32_t blocks = a0.block_end - a0.block_begin;
    if (blocks == 0) return 0;
    SelArgs a = a0;
    a.status_word = ctx->d_status;
    const uint32_t G = a.q_heads / a.kv_heads;
    dim3 grid((blocks + 3u) / 4u, a.kv_heads);
    const size_t qbytes = ((size_t)G * a.hd * sizeof(float) + 127u) & ~(size_t)127u;
    const size_t bulk_smem = qbytes + (size_t)4 * a.block_size * a.hd * sizeof(__half);
    cudaError_t e;
    // staged form: whole 16-byte pieces per block and at most 96 KB per CTA (two or three CTAs per SM)
    if ((a.block_size * a.hd * 2u) % 16u == 0u && bulk_smem <= 96u * 1024u) {
        auto kern = a.hd == 128 ? block_score_bulk_kernel<128> : block_score_bulk_kernel<64>;
        static std::atomic<unsigned long long> configured[2];
        const unsigned long long bit = 1ull << (ctx->device_id & 63);
        std::atomic<unsigned long long>& cfgd = configured[a.hd == 128 ? 1 : 0];
        if (!(cfgd.load(std::memory_order_acquire) & bit)) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) return -8;
            cfgd.fetch_or(bit, std::memory_order_release);
        }
        e = m40_launch_dependent(kern, grid, dim3(128), bulk_smem, ctx->decode_stream, a);
    } else {
        const size_t smem = (size_t)G * a.hd * sizeof(float);
        if (a.hd == 128) e = m40_launch_dependent(block_score_kernel<128>, grid, dim3(128), smem, ctx->decode_stream, a);
        else e = m40_launch_dependent(block_score_kernel<64>, grid, dim3(128), smem, ctx->decode_stream, a);
    }
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// Ranks `r.n` candidates per q head into the top-`r.top_n` list (see rank_topk_kernel). n <= 4096.
int launch_rank(M40llmCudaContext* ctx, const RankArgs& r, uint32_t q_heads) {
    // enough CTAs to spread the n^2 comparisons over the GPU, never more slices than 64-candidate groups
    uint32_t slices = ((uint32_t)ctx->sm_count + q_heads - 1u) / q_heads;
    const uint32_t max_slices = (r.n + 63u) / 64u;
    if (slices > max_slices) slices = max_slices;
    if (slices < 1u) slices = 1u;
    const size_t smem = (size_t)((r.n + 3u) / 4u * 4u + 4u) * 8u;
    const cudaError_t e = m40_launch_dependent(rank_topk_kernel, dim3(q_heads, slices), dim3(256), smem, ctx->decode_stream, r);
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -8;
}

int launch_topk(M40llmCudaContext* ctx, const SelArgs& a) {
    if (a.nb <= 4096u) {
        RankArgs r = {};
        r.scores = a.scores;
        r.ids = nullptr;
        r.out_ids = a.sel_blocks;
        r.out_scores = a.sel_scores;
        r.head_stride = a.score_stride;
        r.part_stride = 0;
        r.per_part = a.nb ? a.nb : 1u;
        r.elem_stride = 1;
        r.n = a.nb;
        r.index_base = 0;
        r.top_n = a.top_n;
        r.out_stride = 1;
        return launch_rank(ctx, r, a.q_heads);
    }
    const size_t smem = (size_t)a.nb * sizeof(float);
    if (smem > 200u * 1024u) return -7;
    if (smem > 48u * 1024u)
        cudaFuncSetAttribute(topk_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_blocks_kernel<<<a.q_heads, 128, smem, ctx->decode_stream>>>(a);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

int launch_attend(M40llmCudaContext* ctx, const SelArgs& a0, bool dense) {
    SelArgs a = a0;
    a.status_word = ctx->d_status;
    cudaStream_t s = ctx->decode_stream;
    cudaError_t e;
    const StagedPlan sp = plan_staged(a, dense, ctx->sm_count);
    if (sp.splits != 0 && sp.splits == a.splits) {  // the caller sized its partials with attend_splits(): same plan
        auto kern = a.hd == 128 ? selected_attend_staged_kernel<128> : selected_attend_staged_kernel<64>;
        const size_t smem = (size_t)sp.warps * sp.slice_bytes;
        static std::atomic<unsigned long long> configured[2];
        const unsigned long long bit = 1ull << (ctx->device_id & 63);
        std::atomic<unsigned long long>& cfgd = configured[a.hd == 128 ? 1 : 0];
        if (!(cfgd.load(std::memory_order_acquire) & bit)) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return -8;
            cfgd.fetch_or(bit, std::memory_order_release);
        }
        e = m40_launch_dependent(kern, dim3(sp.splits, a.q_heads), dim3(32u * sp.warps), smem, s, a, sp.slice_bytes, sp.ring_piece,
                                 sp.ring_items);
        M40_COUNT_LAUNCH(ctx);
        return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -8;
    }
    dim3 grid(a.splits, a.q_heads);
    if (a.hd == 128) {
        if (dense) e = m40_launch_dependent(selected_attend_kernel<128, true>, grid, dim3(128), 0, s, a);
        else e = m40_launch_dependent(selected_attend_kernel<128, false>, grid, dim3(128), 0, s, a);
    } else {
        if (dense) e = m40_launch_dependent(selected_attend_kernel<64, true>, grid, dim3(128), 0, s, a);
        else e = m40_launch_dependent(selected_attend_kernel<64, false>, grid, dim3(128), 0, s, a);
    }
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -8;
}

uint32_t attend_splits(const M40llmCudaContext* ctx, const SelArgs& a, bool dense = false) {
    const StagedPlan sp = plan_staged(a, dense, ctx->sm_count);
    if (sp.splits != 0 && getenv("M40LLM_ATTEND_GATHER") == nullptr) return sp.splits;  // one partial per staged CTA
    const uint32_t total = 64u * a.block_size + (a.seq_len - a.old_len);
    // ~8 CTAs per SM, never fewer than 64 slots per CTA: the kernel is latency-bound, so parallelism is what counts
    uint32_t splits = ((uint32_t)ctx->sm_count * 8u + a.q_heads - 1u) / a.q_heads;
    const uint32_t max_splits = (total + 63u) / 64u;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1u) splits = 1u;
    if (splits > 128u) splits = 128u;
    return splits;
}

// Whole block-select attention for one sequence (selection + attention + merge).
int block_select_attention(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* q,
                           uint32_t q_heads, uint32_t seq_len, uint32_t recent_window, uint32_t block_size,
                           uint32_t top_blocks, void* out, bool dense) {
    if (q_heads > ctx->selected_capacity_heads) return -7;
    SelArgs a = {};
    fill_common(kv, &a, seq_id, q, q_heads, seq_len, recent_window, block_size, top_blocks, dense);
    a.splits = attend_splits(ctx, a, dense);
    const size_t n_scores = (size_t)q_heads * a.score_stride;
    const size_t n_part = (size_t)q_heads * a.splits;
    float* scratch = (float*)m40_ensure_scratch(ctx, 1, (n_scores + n_part * (2 + (size_t)a.hd)) * sizeof(float));
    if (!scratch) return -8;
    a.scores = scratch;
    a.part_m = scratch + n_scores;
    a.part_l = a.part_m + n_part;
    a.part_o = a.part_l + n_part;
    a.sel_blocks = ctx->d_selected_blocks;
    a.sel_scores = ctx->d_selected_scores;
    int rc = launch_scores(ctx, a);
    if (rc != 0) return rc;
    rc = launch_topk(ctx, a);
    if (rc != 0) return rc;
    rc = launch_attend(ctx, a, dense);
    if (rc != 0) return rc;
    return m40_attention_merge_rows(ctx, a.part_m, a.part_l, a.part_o, a.splits, q_heads, a.hd, (float*)out) == 0 ? 0 : -8;
}

// The reference reads its selection policy from the environment inside the hot entry point
// (cuda/kernels.cu:4526-4534). Only the default policy (top-k, score order) is implemented;
// any other setting is refused instead of silently differing.
bool non_default_policy_requested() {
    const char* p = getenv("M40LLM_KV_BLOCK_SELECT_POLICY");
    if (p && p[0] != '\0' && strcmp(p, "topk") != 0) return true;
    const char* o = getenv("M40LLM_KV_SELECTED_BLOCK_ORDER");
    if (o && o[0] != '\0' && strcmp(o, "score") != 0) return true;
    return false;
}

}  // namespace

extern "C" {

int m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;
    if (!kv->fp16_k_q4_v_backing || !kv->d_old_k || !kv->d_q4_v || !kv->d_q4_scale || !kv->d_recent_k ||
        !kv->d_recent_v)
        return -16;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -4;
    if (kv->head_dim != 64 && kv->head_dim != 128) return -5;
    if (recent_window == 0 || block_size == 0 || top_blocks == 0 || top_blocks > 64) return -6;
    // The ring is addressed with the cache's own window (kernels.cu:3036 uses the argument for both;
    // the reference host always passes the cache's configuration, src/infer/kv.rs:562-575).
    if (recent_window != kv->recent_window) return -6;
    if (non_default_policy_requested()) return M40LLM_ERR_UNSUPPORTED;
    if (m40_ensure_device(ctx) != 0) return -1;
    return block_select_attention(ctx, kv, seq_id, d_q_f32, q_heads, seq_len, recent_window, block_size, top_blocks,
                                  d_out_f32, false);
}

int m40llm_attention_last_token_f32_gqa_block_select_exact_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                                 uint32_t seq_id, const void* d_q_f32,
                                                                 uint32_t q_heads, uint32_t seq_len,
                                                                 uint32_t recent_window, uint32_t block_size,
                                                                 uint32_t top_blocks, void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -4;
    if (kv->head_dim != 64 && kv->head_dim != 128) return -5;
    if (recent_window == 0 || block_size == 0 || top_blocks == 0 || top_blocks > 64) return -6;
    if (!kv->d_k || !kv->d_v) return -7;
    if (non_default_policy_requested()) return M40LLM_ERR_UNSUPPORTED;
    if (m40_ensure_device(ctx) != 0) return -1;
    return block_select_attention(ctx, kv, seq_id, d_q_f32, q_heads, seq_len, recent_window, block_size, top_blocks,
                                  d_out_f32, true);
}

int m40llm_kvcache_score_old_blocks_async(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                          const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                          uint32_t block_begin, uint32_t block_end, void* d_scores_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_scores_f32) return -1;
    if (!kv->compressed || !kv->d_old_k) return -16;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -4;
    if (kv->head_dim != 64 && kv->head_dim != 128) return -5;
    if (m40_ensure_device(ctx) != 0) return -1;
    SelArgs a = {};
    fill_common(kv, &a, seq_id, d_q_f32, q_heads, seq_len, kv->recent_window, kv->block_size, 64, false);
    if (block_begin > block_end || block_end > a.nb) return -6;
    a.block_begin = block_begin;
    a.block_end = block_end;
    a.score_stride = block_end - block_begin ? block_end - block_begin : 1u;
    a.scores = (float*)d_scores_f32;
    return launch_scores(ctx, a);
}

int m40llm_attention_compressed_selected_partial_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                       uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                       uint32_t seq_len, const uint32_t* d_blocks,
                                                       uint32_t block_begin, uint32_t block_end,
                                                       uint32_t include_recent, void* d_m_f32, void* d_l_f32,
                                                       void* d_o_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_blocks || !d_m_f32 || !d_l_f32 || !d_o_f32) return -1;
    if (!kv->compressed || !kv->d_old_k || !kv->d_q4_v) return -16;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -4;
    if (kv->head_dim != 64 && kv->head_dim != 128) return -5;
    if (m40_ensure_device(ctx) != 0) return -1;
    SelArgs a = {};
    fill_common(kv, &a, seq_id, d_q_f32, q_heads, seq_len, kv->recent_window, kv->block_size, 64, false);
    if (block_begin > block_end || block_end > a.nb) return -6;
    a.block_begin = block_begin;
    a.block_end = block_end;
    a.include_recent = include_recent ? 1u : 0u;
    a.sel_blocks = const_cast<uint32_t*>(d_blocks);
    a.splits = attend_splits(ctx, a);
    const size_t n_part = (size_t)q_heads * a.splits;
    float* scratch = (float*)m40_ensure_scratch(ctx, 1, n_part * (2 + (size_t)a.hd) * sizeof(float));
    if (!scratch) return -8;
    a.part_m = scratch;
    a.part_l = scratch + n_part;
    a.part_o = scratch + 2 * n_part;
    int rc = launch_attend(ctx, a, false);
    if (rc != 0) return rc;
    return m40_attention_fold_partials(ctx, a.part_m, a.part_l, a.part_o, a.splits, q_heads, a.hd, (float*)d_m_f32,
                                       (float*)d_l_f32, (float*)d_o_f32) == 0 ? 0 : -8;
}

int m40llm_topk_pairs_async(M40llmCudaContext* ctx, const void* d_scores_f32, uint32_t q_heads, uint32_t n,
                            uint32_t score_stride, uint32_t index_base, uint32_t top_n, void* d_pairs_out) {
    if (!ctx || !d_scores_f32 || !d_pairs_out) return -1;
    if (q_heads == 0 || top_n == 0 || top_n > 64 || n > 4096 || score_stride < n) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    RankArgs r = {};
    r.scores = (const float*)d_scores_f32;
    r.out_scores = (float*)d_pairs_out;
    r.out_ids = (uint32_t*)d_pairs_out + 1;
    r.head_stride = score_stride;
    r.per_part = n ? n : 1u;
    r.elem_stride = 1;
    r.n = n;
    r.index_base = index_base;
    r.top_n = top_n;
    r.out_stride = 2;
    return launch_rank(ctx, r, q_heads);
}

int m40llm_topk_merge_pairs_async(M40llmCudaContext* ctx, const void* d_pairs, uint32_t parts, uint32_t q_heads,
                                  uint32_t top_n, uint32_t* d_blocks_out, void* d_scores_out_f32) {
    if (!ctx || !d_pairs || !d_blocks_out) return -1;
    if (q_heads == 0 || parts == 0 || top_n == 0 || top_n > 64 || parts > 64) return -2;
    if (q_heads > ctx->selected_capacity_heads) return -7;
    if (m40_ensure_device(ctx) != 0) return -1;
    RankArgs r = {};
    r.scores = (const float*)d_pairs;
    r.ids = (const uint32_t*)d_pairs + 1;
    r.out_ids = d_blocks_out;
    r.out_scores = d_scores_out_f32 ? (float*)d_scores_out_f32 : ctx->d_selected_scores;
    r.head_stride = 64u * 2u;
    r.part_stride = (size_t)q_heads * 64u * 2u;
    r.per_part = 64;
    r.elem_stride = 2;
    r.n = parts * 64u;
    r.top_n = top_n;
    r.out_stride = 1;
    return launch_rank(ctx, r, q_heads);
}

int m40llm_kvcache_debug_last_selected_blocks(M40llmCudaContext* ctx, uint32_t q_heads, uint32_t* out_blocks_host,
                                              float* out_scores_host) {
    if (!ctx || !out_blocks_host) return -1;
    if (q_heads == 0 || q_heads > ctx->selected_capacity_heads) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    if (cudaStreamSynchronize(ctx->decode_stream) != cudaSuccess) return -3;
    if (cudaMemcpy(out_blocks_host, ctx->d_selected_blocks, (size_t)q_heads * 64 * sizeof(uint32_t),
                   cudaMemcpyDeviceToHost) != cudaSuccess)
        return -4;
    if (out_scores_host && cudaMemcpy(out_scores_host, ctx->d_selected_scores, (size_t)q_heads * 64 * sizeof(float),
                                      cudaMemcpyDeviceToHost) != cudaSuccess)
        return -4;
    return 0;
}

int m40llm_kvcache_debug_select_old_blocks(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                           const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                           uint32_t recent_window, uint32_t block_size, uint32_t top_blocks,
                                           uint32_t* out_blocks_host, float* out_scores_host, uint32_t* out_start_host,
                                           uint32_t* out_end_host, uint32_t* out_count, uint32_t max_out,
                                           uint32_t* out_total_old_blocks) {
    if (!ctx || !kv || !d_q_f32 || !out_blocks_host || !out_scores_host || !out_start_host || !out_end_host ||
        !out_count || !out_total_old_blocks)
        return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (q_heads == 0 || kv->num_heads == 0 || kv->head_dim == 0) return -3;
    if (seq_len == 0 || seq_len > kv->max_seq_len || block_size == 0 || max_out == 0) return -4;
    const uint32_t eff_recent = kv->compressed ? kv->recent_window : recent_window;
    const uint32_t eff_block = kv->compressed ? kv->block_size : block_size;
    if (eff_recent == 0 || eff_block == 0) return -5;
    if (kv->head_dim != 64 && kv->head_dim != 128) return -3;
    if (q_heads % kv->num_heads != 0) return -3;
    if (non_default_policy_requested()) return M40LLM_ERR_UNSUPPORTED;
    if (m40_ensure_device(ctx) != 0) return -1;
    const bool dense = !kv->compressed;
    if (dense && !kv->d_k) return -9;
    if (!dense && !kv->d_old_k) return -12;
    SelArgs a = {};
    fill_common(kv, &a, seq_id, d_q_f32, q_heads, seq_len, eff_recent, eff_block, 64, dense);
    *out_total_old_blocks = a.nb;
    *out_count = 0;
    if (a.nb == 0) return 0;
    uint32_t want = top_blocks == 0 ? a.nb : (top_blocks < a.nb ? top_blocks : a.nb);
    if (want > max_out) want = max_out;
    if (want > 64u) want = 64u;
    a.top_n = want;
    float* scratch = (float*)m40_ensure_scratch(ctx, 1, (size_t)q_heads * a.score_stride * sizeof(float));
    if (!scratch) return -6;
    a.scores = scratch;
    a.sel_blocks = ctx->d_selected_blocks;
    a.sel_scores = ctx->d_selected_scores;
    if (launch_scores(ctx, a) != 0 || launch_topk(ctx, a) != 0) return -6;
    if (cudaStreamSynchronize(ctx->decode_stream) != cudaSuccess) return -6;
    uint32_t blocks[64];
    float scores[64];
    // the reference reports q head 0 / kv head 0 only (kernels.cu:6485-6486, 6533)
    if (cudaMemcpy(blocks, ctx->d_selected_blocks, sizeof(blocks), cudaMemcpyDeviceToHost) != cudaSuccess) return -7;
    if (cudaMemcpy(scores, ctx->d_selected_scores, sizeof(scores), cudaMemcpyDeviceToHost) != cudaSuccess) return -7;
    uint32_t n = 0;
    for (uint32_t i = 0; i < want; ++i) {
        if (blocks[i] == 0xffffffffu) continue;
        const uint32_t start = blocks[i] * eff_block;
        const uint32_t end = start + eff_block < a.old_len ? start + eff_block : a.old_len;
        out_blocks_host[n] = blocks[i];
        out_scores_host[n] = scores[i];
        out_start_host[n] = start;
        out_end_host[n] = end;
        ++n;
    }
    *out_count = n;
    return 0;
}

// ---- compressed-cache modes outside the decode hot path ----
#define M40_UNSUPPORTED_SELECT_BODY                                                          \
    (void)recent_window; (void)block_size; (void)top_blocks;                                  \
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;                                     \
    if (seq_id >= kv->max_batch_size) return -2;                                              \
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;                                 \
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -4;        \
    return M40LLM_ERR_UNSUPPORTED;

int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32) {
    M40_UNSUPPORTED_SELECT_BODY
}
int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_with_buffers_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* staged_k_dev,
    void* staged_v_dev, void* staged_positions_dev, void* staged_counts_dev, uint32_t staged_capacity_tokens,
    void* d_out_f32) {
    (void)staged_k_dev; (void)staged_v_dev; (void)staged_positions_dev; (void)staged_counts_dev;
    (void)staged_capacity_tokens;
    M40_UNSUPPORTED_SELECT_BODY
}
int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_q8_old_with_buffers_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* staged_k_dev,
    void* staged_v_dev, void* staged_positions_dev, void* staged_counts_dev, uint32_t staged_capacity_tokens,
    void* d_out_f32) {
    (void)staged_k_dev; (void)staged_v_dev; (void)staged_positions_dev; (void)staged_counts_dev;
    (void)staged_capacity_tokens;
    M40_UNSUPPORTED_SELECT_BODY
}
int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_fp16_k_q4_v_old_with_buffers_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* staged_k_dev,
    void* staged_v_dev, void* staged_positions_dev, void* staged_counts_dev, uint32_t staged_capacity_tokens,
    void* d_out_f32) {
    (void)staged_k_dev; (void)staged_v_dev; (void)staged_positions_dev; (void)staged_counts_dev;
    (void)staged_capacity_tokens;
    M40_UNSUPPORTED_SELECT_BODY
}
int m40llm_attention_last_token_f32_gqa_block_select_exact_q8_old_direct_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32) {
    M40_UNSUPPORTED_SELECT_BODY
}
int m40llm_attention_last_token_f32_gqa_block_summary_lossy_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32) {
    M40_UNSUPPORTED_SELECT_BODY
}
int m40llm_attention_last_token_f32_gqa_compressed_recent_only_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                                     uint32_t seq_id, const void* d_q_f32,
                                                                     uint32_t q_heads, uint32_t seq_len,
                                                                     void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;
    if (!kv->compressed) return -2;
    if (seq_id >= kv->max_batch_size) return -3;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -4;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -5;
    return M40LLM_ERR_UNSUPPORTED;
}

}  // extern "C"
