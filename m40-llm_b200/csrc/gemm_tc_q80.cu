// Batched decode projections over Q8_0 GGUF rows on the tcgen05 tensor cores.
//
// Q8_0 stores 32 weights as {f16 d; int8 q[32]} (34 bytes, cuda/kernels.cu:856-867 of the reference):
// w = d * q with a different d for every (row, 32-k block).
//
//   raw bytes   TMA (plain 2D box of 128 rows x 272 bytes = 8 blocks per row) straight from the GGUF layout, four
//               stages deep;
//   dequant     16 worker warps. Worker group g (4 warps = 128 threads = 128 weight rows) owns the g-th 64-k
//               sub-block of every raw stage; a thread turns the two blocks of its row into TWO f16 operands,
//               hi = rn(d*q) and lo = d*q - hi (exact by FMA), so hi + lo carries the product to ~2^-22 -- the value
//               the reference computes in f32 -- and stores them with tcgen05.st straight into TENSOR MEMORY
//               (lane = weight row, one column = two f16 along k). No shared-memory round trip for the converted
//               operand, and the operand ring is seven sub-blocks deep;
//   MMA         D[128 x M_pad] += hi.Xh + hi.Xl + lo.Xh with the A operand read from tensor memory and the
//               activations (split the same way) from shared memory, f32 accumulators in TMEM, one accumulator per
//               tile segment (two alternate between segments). One thread can issue a tcgen05.mma (or commit) only
//               every ~45 cycles whatever its width, while the tensor core needs ~33 + 16 cycles for a 128 x 16 weight
//               operand against 64 + 32 activation columns: with one issuing thread the kernel is issue-bound. Up to
//               32 rows two threads issue side by side, one the hi.[Xh | Xl] products and one the lo.Xh products,
//               into separate accumulator columns (no ordering between the two is needed), and each sub-block is
//               committed once per thread to ONE completion barrier that frees both the operand stage and the
//               activation slot;
//   epilogue    the worker threads read their row of D back (tcgen05.ld) at the end of a segment.
//
// Work is split stream-K style: the (tile, 256-k unit) space is cut into one contiguous span per CTA (one CTA per
// SM), so every SM streams the same number of weight bytes. A span that crosses tile boundaries writes one partial
// per tile; the epilogue kernel adds the partials of each tile and applies residual or SiLU(gate)*up.
//
// Every wait is bounded; a wait that runs out sets bit 4 of the context's device status word and the CTA
// drains, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace {

using namespace tc;

constexpr uint32_t UNIT_K = 256;                       // k per raw stage (8 Q8_0 blocks)
constexpr uint32_t RAW_ROW_BYTES = UNIT_K / 32 * 34;   // 272
constexpr uint32_t RAW_BYTES = BLOCK_N * RAW_ROW_BYTES; // 34816
constexpr uint32_t RS = 4;                             // raw stages
constexpr uint32_t A_COLS = BLOCK_K;                   // TMEM columns of one converted sub-block: 32 hi + 32 lo
constexpr uint32_t TMEM_COLS = 512;
// Two issuing threads (see above), the lo.Xh products in a column group of their own. Up to 32 rows two accumulator
// sets alternate between tile segments; at 64 rows the three column groups leave room for one set only (the issue
// then waits at a segment boundary until the workers have read it, ~1 us per call), which still beats one thread
// issuing all eight instructions of a sub-block.
__host__ __device__ constexpr bool dual_issue(int m_pad) { return m_pad <= 64; }
__host__ __device__ constexpr uint32_t acc_sets(int m_pad) { return m_pad <= 32 ? 2u : 1u; }
__host__ __device__ constexpr uint32_t n_issuers(int m_pad) { return dual_issue(m_pad) ? 2u : 1u; }
// dual: [hi.Xh | hi.Xl | lo.Xh]; single: [hi.Xh + lo.Xh | hi.Xl]
__host__ __device__ constexpr uint32_t acc_cols(int m_pad) { return (dual_issue(m_pad) ? 3u : 2u) * (uint32_t)m_pad; }
__host__ __device__ constexpr uint32_t a_stages(int m_pad) { return (TMEM_COLS - acc_sets(m_pad) * acc_cols(m_pad)) / A_COLS; }  // 6, 5, 5
// First TMEM column of accumulator set tb. Every accumulator starts at a multiple of its own width:
// dual issue lays the two buffers out as [hi 0 | lo 0 | lo 1 | hi 1] with hi 2 m_pad and lo m_pad columns wide.
__host__ __device__ constexpr uint32_t acc_hi_col(int m_pad, uint32_t tb) {
    return dual_issue(m_pad) ? (tb ? 4u * (uint32_t)m_pad : 0u) : tb * acc_cols(m_pad);
}
__host__ __device__ constexpr uint32_t acc_lo_col(int m_pad, uint32_t tb) { return (2u + tb) * (uint32_t)m_pad; }  // dual only
// Activation tiles: their bytes are counted on the operand stage's barrier, but they live in a ring of their own that
// is a few slots deeper, so that a tile is requested when its stage's previous use has been ISSUED, not completed.
// The completion barriers form a ring of the same depth: done[u % b_slots] flips when every MMA of sub-block u has
// finished, which frees activation slot u % b_slots at once and operand stage u % a_stages for sub-block u + a_stages.
__host__ __device__ constexpr uint32_t b_slots(int m_pad) { return a_stages(m_pad) + (m_pad <= 32 ? 3u : 0u); }

struct Q80Args {
    float* partial;  // [ctas][seg_max][M][128]
    uint32_t* status;
    uint32_t M, K;
    uint32_t tile_begin[4], problems, tiles_total;
    uint32_t units_per_tile;  // K / 256
    uint32_t units_total, ctas, seg_max;
};

__device__ __forceinline__ void span_of(const Q80Args& a, uint32_t cta, uint32_t* u0, uint32_t* u1) {
    // units_total * ctas < 2^32 is checked on the host: 32-bit divisions
    *u0 = (cta * a.units_total) / a.ctas;
    *u1 = ((cta + 1u) * a.units_total) / a.ctas;
}

struct Q80Smem {
    unsigned char* s_raw;
    uint64_t *raw_full, *raw_empty, *a_full, *done, *t_full, *t_empty;
    volatile uint32_t* abort_flag;
};

constexpr uint32_t WORKER_WARPS = 16;                    // 4 threads per weight row
constexpr uint32_t WORKER_THREADS = WORKER_WARPS * 32;   // 512
constexpr uint32_t SERVICE_WARPS = 4;                    // weight producer, MMA issuer, activation producer, 2nd issuer
constexpr uint32_t CTA_THREADS = SERVICE_WARPS * 32 + WORKER_THREADS;

// One worker thread owns weight row r of the tile and, in every raw stage, the C4-th 64-k sub-block (two Q8_0
// blocks, bytes [68*C4, 68*C4+68) of the row: 4-byte aligned). At the end of a tile segment it reads columns
// [C4*M_PAD/4, +M_PAD/4) of its row of the accumulator.
template <int M_PAD, int C4>
__device__ __forceinline__ void q80_worker(const Q80Args& a, const Q80Smem& sm, uint32_t tmem_base, uint32_t u0,
                                           uint32_t u1, uint32_t lane_group, uint32_t lane) {
    constexpr int COLS = M_PAD / 4;
    constexpr uint32_t AST = a_stages(M_PAD), BS = b_slots(M_PAD), TB = acc_sets(M_PAD);
    constexpr uint32_t A_COL0 = TB * acc_cols(M_PAD);
    const uint32_t r = lane_group * 32 + lane;  // weight row of the tile == TMEM lane
    const uint32_t tmem_lane = tmem_base + ((lane_group * 32u) << 16);
    bool ok = true;
    uint32_t icount = 0;  // raw stages consumed by this CTA so far
    // every wait of a worker warp is made warp-uniform so the warp-collective tcgen05 instructions stay converged
    auto wwait = [&](uint64_t* bar, uint32_t parity) {
        const bool r0 = mbar_wait(bar, parity);
        return (bool)__all_sync(0xffffffffu, r0);
    };
    uint32_t pos = u0, seg = 0;
    while (pos < u1 && ok) {
        const uint32_t kb_begin = pos % a.units_per_tile;
        uint32_t kb_end = kb_begin + (u1 - pos);
        if (kb_end > a.units_per_tile) kb_end = a.units_per_tile;
        for (uint32_t kb = kb_begin; kb < kb_end && ok; ++kb, ++icount) {
            const uint32_t rs = icount % RS;
            const uint32_t u = icount * 4u + C4, as = u % AST;  // this group's sub-block and its operand stage
            if (!wwait(&sm.raw_full[rs], (icount / RS) & 1u)) { ok = false; break; }
            // 68 bytes = words [C4, C4+17) of the five 16-byte chunks that cover them; the row pitch is 17 chunks,
            // so the 16-byte reads of a warp's 32 rows fall on distinct banks
            const uint4* chunk = reinterpret_cast<const uint4*>(sm.s_raw + rs * RAW_BYTES + r * RAW_ROW_BYTES) + (68 * C4) / 16;
            uint32_t L[20];
#pragma unroll
            for (int i = 0; i < 5; ++i) {
                const uint4 t = chunk[i];
                L[4 * i] = t.x, L[4 * i + 1] = t.y, L[4 * i + 2] = t.z, L[4 * i + 3] = t.w;
            }
            // The raw bytes of this stage are in registers now: the slot goes back to the weight producer at once, not
            // after the (long) wait for a free operand stage below, so that the next raw stage is requested a whole
            // conversion earlier. The arrive carries a value computed from every loaded chunk, which makes it wait
            // for the loads themselves (a warp's shared-memory load completes for all its lanes together).
            {
                const uint32_t seen = L[0] ^ L[4] ^ L[8] ^ L[12] ^ L[16] ^ L[3] ^ L[7] ^ L[11] ^ L[15] ^ L[19];
                __syncwarp();
                if (lane == 0)
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0]; // %1" ::"r"(smem_u32(&sm.raw_empty[rs])), "r"(seen) : "memory");
            }
            // the stage is free once every MMA of the sub-block that used it last (u - AST) has completed
            if (u >= AST && !wwait(&sm.done[(u - AST) % BS], ((u - AST) / BS) & 1u)) { ok = false; break; }
            tc_fence_after();
            const __half2 bias = __float2half2_rn(1152.0f);
            const uint32_t col = tmem_lane + A_COL0 + as * A_COLS;
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                // block 0: scale in the low half of word 0, weights from byte 2; block 1: scale in the high half
                // of word 8, weights word aligned from word 9
                const uint32_t dbits = blk == 0 ? (L[C4] & 0xffffu) : (L[C4 + 8] >> 16);
                const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint32_t word = blk == 0 ? __funnelshift_r(L[C4 + j], L[C4 + j + 1], 16) : L[C4 + 9 + j];
                    word ^= 0x80808080u;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t y = __byte_perm(word, 0x64646464u, h ? 0x7362 : 0x5140);  // (1024+u0, 1024+u1)
                        const __half2 q2 = __hsub2(*reinterpret_cast<const __half2*>(&y), bias);  // exact ints
                        const __half2 h2 = __hmul2(q2, d2);                                       // rn(d*q)
                        const __half2 l2 = __hfma2(q2, d2, __hneg2(h2));                          // d*q - hi, exact
                        hi[2 * j + h] = *reinterpret_cast<const uint32_t*>(&h2);
                        lo[2 * j + h] = *reinterpret_cast<const uint32_t*>(&l2);
                    }
                }
                tmem_st_x16(col + blk * 16, hi);
                tmem_st_x16(col + 32 + blk * 16, lo);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.a_full[as]);
        }
        if (!ok) break;
        // ---- end of the tile segment: read this row's accumulator columns and store the partial
        const uint32_t tb = seg % TB;
        if (!wwait(&sm.t_full[tb], (seg / TB) & 1u)) { ok = false; break; }
        tc_fence_after();
        uint32_t x[COLS], y[COLS], z[COLS];
        const uint32_t tlane = tmem_base + ((lane_group * 32u) << 16) + C4 * COLS;
        const uint32_t taddr = tlane + acc_hi_col(M_PAD, tb);
        if (COLS == 4) { tmem_ld_x4(taddr, x); tmem_ld_x4(taddr + M_PAD, y); }
        else if (COLS == 8) { tmem_ld_x8(taddr, x); tmem_ld_x8(taddr + M_PAD, y); }
        else { tmem_ld_x16(taddr, x); tmem_ld_x16(taddr + M_PAD, y); }
        if (dual_issue(M_PAD)) {  // the lo.Xh products have their own column group
            if (COLS == 4) tmem_ld_x4(tlane + acc_lo_col(M_PAD, tb), z);
            else if (COLS == 8) tmem_ld_x8(tlane + acc_lo_col(M_PAD, tb), z);
            else tmem_ld_x16(tlane + acc_lo_col(M_PAD, tb), z);
        }
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.t_empty[tb]);
        float* dstp = a.partial + ((size_t)(blockIdx.x * a.seg_max + seg) * a.M) * BLOCK_N + r;
#pragma unroll
        for (int j = 0; j < COLS; ++j) {
            const uint32_t m = C4 * COLS + j;
            float v = __uint_as_float(x[j]) + __uint_as_float(y[j]);
            if (dual_issue(M_PAD)) v += __uint_as_float(z[j]);
            if (m < a.M) dstp[(size_t)m * BLOCK_N] = v;
        }
        pos += kb_end - kb_begin;
        ++seg;
    }
    if (!ok) *sm.abort_flag = 1;
}

// One MMA-issuing thread. ROLE 0: both products of a sub-block (single issuer); 1: hi.[Xh | Xl]; 2: lo.Xh into its
// own accumulator columns. The loop is this kernel's critical path: stage index and phase are carried, not
// recomputed, and every instantiation holds only the instructions of its own role.
template <int M_PAD, int ROLE>
__device__ __forceinline__ void q80_issuer(const Q80Args& a, const Q80Smem& sm, uint32_t tmem_base, uint32_t b_smem0,
                                        uint32_t u0, uint32_t u1) {
    constexpr uint32_t B_BYTES = M_PAD * BLOCK_K * 2;
    constexpr uint32_t BS = b_slots(M_PAD), AST = a_stages(M_PAD), TB = acc_sets(M_PAD);
    constexpr uint32_t A_COL0 = TB * acc_cols(M_PAD);
    const uint32_t idesc2 = make_idesc(2 * M_PAD), idesc1 = make_idesc(M_PAD);
    bool ok = true;
    uint32_t pos = u0, seg = 0, as = 0, ph = 0, bs = 0;
    const uint32_t a_tmem0 = tmem_base + A_COL0;
    // Everything the loop needs per sub-block is carried as a running value (barrier addresses, the operand's
    // tensor-memory column, the activation descriptor, whose address field counts 16-byte units): the thread's few
    // dozen dependent instructions per sub-block are what this kernel waits for.
    const uint64_t b_desc0 = make_desc_sw128(b_smem0);
    const uint32_t a_full0 = smem_u32(sm.a_full), done0 = smem_u32(sm.done);
    uint32_t a_bar = a_full0, d_bar = done0, ta = a_tmem0 + (ROLE == 2 ? 32u : 0u);
    uint64_t b_x = b_desc0;
    auto wait_bar = [](uint32_t addr, uint32_t parity) {
        for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
            uint32_t done;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done) : "r"(addr), "r"(parity) : "memory");
            if (done) return true;
        }
        return false;
    };
    while (pos < u1 && ok) {
        const uint32_t kb_begin = pos % a.units_per_tile;
        uint32_t kb_end = kb_begin + (u1 - pos);
        if (kb_end > a.units_per_tile) kb_end = a.units_per_tile;
        const uint32_t tb = seg % TB;
        if (seg >= TB && !mbar_wait(&sm.t_empty[tb], ((seg / TB) - 1) & 1u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (ROLE == 2 ? acc_lo_col(M_PAD, tb) : acc_hi_col(M_PAD, tb));
        const uint32_t n_sub = (kb_end - kb_begin) * 4;
        uint32_t acc = 0u;  // 0 only for the first MMA of the segment
        for (uint32_t j = 0; j < n_sub; ++j) {
            if (!wait_bar(a_bar, ph)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (uint32_t kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
                // rows [0, M_PAD) of the activation tile = Xh, [M_PAD, 2 M_PAD) = Xl
                const uint64_t b_k = b_x + (uint64_t)((kk * UMMA_K * 2) >> 4);
                const uint32_t a_k = ta + kk * (UMMA_K / 2);  // hi columns [0,32), lo columns [32,64) of the stage
                if (ROLE == 2) {
                    umma_f16_ts(d_tmem, a_k, b_k, idesc1, acc | kk);
                } else {
                    umma_f16_ts(d_tmem, a_k, b_k, idesc2, acc | kk);
                    if (ROLE == 0) umma_f16_ts(d_tmem, a_k + 32, b_k, idesc1, 1u);
                }
            }
            acc = 1u;
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(d_bar) : "memory");
            // this thread's share of sub-block done: operand stage and activation slot
            ++as, a_bar += 8u, ta += A_COLS;
            if (as == AST) as = 0, ph ^= 1u, a_bar = a_full0, ta -= AST * A_COLS;
            ++bs, d_bar += 8u, b_x += (uint64_t)((2 * B_BYTES) >> 4);
            if (bs == BS) bs = 0, d_bar = done0, b_x = b_desc0;
        }
        if (ok) umma_commit(&sm.t_full[tb]);
        pos += kb_end - kb_begin;
        ++seg;
    }
    if (!ok) *sm.abort_flag = 1;
}

template <int M_PAD>
__global__ void __launch_bounds__(CTA_THREADS, 1) gemm_tc_q80_kernel(const __grid_constant__ CUtensorMap tmW0,
                                                                     const __grid_constant__ CUtensorMap tmW1,
                                                                     const __grid_constant__ CUtensorMap tmW2,
                                                                     const __grid_constant__ CUtensorMap tmXh,
                                                                     const __grid_constant__ CUtensorMap tmXl,
                                                                     Q80Args a) {
    constexpr uint32_t B_BYTES = M_PAD * BLOCK_K * 2;  // one of hi / lo for a 64-k sub-block
    constexpr uint32_t BS = b_slots(M_PAD), TB = acc_sets(M_PAD);
    constexpr uint32_t AST = a_stages(M_PAD);
    constexpr uint32_t A_COL0 = TB * acc_cols(M_PAD);
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    unsigned char* s_raw = smem;                             // RS x RAW_BYTES
    unsigned char* s_b = s_raw + RS * RAW_BYTES;             // BS x (hi, lo); 1024-aligned: RAW_BYTES = 34 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_b + BS * 2 * B_BYTES);
    constexpr uint32_t NI = n_issuers(M_PAD);
    uint64_t* raw_full = bars;
    uint64_t* raw_empty = raw_full + RS;
    uint64_t* a_full = raw_empty + RS;
    uint64_t* done = a_full + AST;
    uint64_t* t_full = done + BS;
    uint64_t* t_empty = t_full + TB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(t_empty + TB);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

    uint32_t u0, u1;
    span_of(a, blockIdx.x, &u0, &u1);
    const uint32_t n_units = u1 - u0;

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < RS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], WORKER_WARPS); }
        // a stage is full when its 4 worker warps have arrived AND the activation tile's bytes have landed (the
        // activation producer's expect_tx is the fifth arrival); one commit frees it for both
        for (uint32_t i = 0; i < AST; ++i) mbar_init(&a_full[i], 5);
        for (uint32_t i = 0; i < BS; ++i) mbar_init(&done[i], NI);  // one commit per issuing thread
        for (uint32_t i = 0; i < TB; ++i) { mbar_init(&t_full[i], NI); mbar_init(&t_empty[i], WORKER_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------- weight producer (weights never depend on the previous kernel: no dependency wait here): raw Q8_0 stages, running up to RS units ahead of the workers
        if (lane == 0) {
            bool ok = true;
            for (uint32_t i = 0; i < n_units && ok; ++i) {
                const uint32_t unit = u0 + i;
                const uint32_t tile = unit / a.units_per_tile, kb = unit % a.units_per_tile;
                uint32_t p = 0;
                while (p + 1 < a.problems && tile >= a.tile_begin[p + 1]) ++p;
                const CUtensorMap* tmW = p == 0 ? &tmW0 : (p == 1 ? &tmW1 : &tmW2);
                const uint32_t row0 = (tile - a.tile_begin[p]) * BLOCK_N;
                const uint32_t rs = i % RS;
                if (i >= RS && !mbar_wait(&raw_empty[rs], ((i / RS) - 1) & 1u)) { ok = false; break; }
                if (*abort_flag) { ok = false; break; }
                mbar_expect_tx(&raw_full[rs], RAW_BYTES);
                tma_load_2d(s_raw + rs * RAW_BYTES, tmW, &raw_full[rs], (int)(kb * (RAW_ROW_BYTES / 2)), (int)row0);
            }
            if (!ok) *abort_flag = 1;
        }
    } else if (warp == 2) {
        // ---------------- activation producer: hi and lo f16 copies of X for every 64-k sub-block
        if (lane == 0) {
            pdl_wait();  // X was split by the previous kernel
            bool ok = true;
            for (uint32_t i = 0; i < n_units && ok; ++i) {
                const uint32_t kb = (u0 + i) % a.units_per_tile;
                for (uint32_t sub = 0; sub < 4; ++sub) {
                    const uint32_t u = i * 4 + sub, as = u % AST, bs = u % BS;
                    // the slot must be free (the MMAs of sub-block u - BS have completed) and the stage barrier must
                    // have finished its previous use (sub-block u - AST was handed to the MMA issuer)
                    if (u >= BS && !mbar_wait(&done[bs], ((u / BS) - 1) & 1u)) { ok = false; break; }
                    if (u >= AST && !mbar_wait(&a_full[as], ((u / AST) - 1) & 1u)) { ok = false; break; }
                    if (*abort_flag) { ok = false; break; }
                    mbar_expect_tx(&a_full[as], 2 * B_BYTES);
                    const int kx = (int)(kb * UNIT_K + sub * BLOCK_K);
                    tma_load_2d(s_b + bs * 2 * B_BYTES, &tmXh, &a_full[as], kx, 0);
                    tma_load_2d(s_b + bs * 2 * B_BYTES + B_BYTES, &tmXl, &a_full[as], kx, 0);
                }
            }
            if (!ok) *abort_flag = 1;
        }
    } else if (warp == 1 || warp == 3) {
        // ---------------- MMA issuers: one accumulator per tile segment, TMEM buffer = segment % TB. Warp 1 issues
        // hi against [Xh | Xl] (the two activation tiles are contiguous rows of one operand); the lo.Xh products go
        // to warp 3 and their own accumulator columns (dual issue) or follow from warp 1 into the first half.
        // The two roles are separate instantiations: with both products under a run-time condition in one loop the
        // compiler predicated them, and a predicated-off tcgen05.mma still costs its ~70-90 cycles in the issue slot.
        if (lane == 0) {
            Q80Smem sm = {s_raw, raw_full, raw_empty, a_full, done, t_full, t_empty, abort_flag};
            if (!dual_issue(M_PAD)) {
                if (warp == 1) q80_issuer<M_PAD, 0>(a, sm, tmem_base, smem_u32(s_b), u0, u1);
            } else if (warp == 1) {
                q80_issuer<M_PAD, 1>(a, sm, tmem_base, smem_u32(s_b), u0, u1);
            } else {
                q80_issuer<M_PAD, 2>(a, sm, tmem_base, smem_u32(s_b), u0, u1);
            }
        }
    } else {
        // ---------------- workers: warps 4..19; TMEM lane group = warp % 4, k quarter of a raw stage = (warp - 4) / 4
        Q80Smem sm = {s_raw, raw_full, raw_empty, a_full, done, t_full, t_empty, abort_flag};
        pdl_wait();  // the partials written at segment ends reuse scratch that earlier kernels may still read
        const uint32_t lane_group = warp & 3u;
        switch ((warp - SERVICE_WARPS) >> 2) {
            case 0: q80_worker<M_PAD, 0>(a, sm, tmem_base, u0, u1, lane_group, lane); break;
            case 1: q80_worker<M_PAD, 1>(a, sm, tmem_base, u0, u1, lane_group, lane); break;
            case 2: q80_worker<M_PAD, 2>(a, sm, tmem_base, u0, u1, lane_group, lane); break;
            default: q80_worker<M_PAD, 3>(a, sm, tmem_base, u0, u1, lane_group, lane); break;
        }
    }
    if (*abort_flag && threadIdx.x == SERVICE_WARPS * 32) atomicOr(a.status, 4u);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

struct Q80EpiArgs {
    const float* partial;
    __half* split_hi;  // optional (mode 1): the result as f16 hi | lo copies for a following tensor-core call
    __half* split_lo;
    float* out[3];
    const float* residual[3];
    uint32_t N[3];
    uint32_t tile_begin[4];
    uint32_t M, units_per_tile, units_total, ctas, seg_max, mode, problems;
};

// The CTAs whose spans hold a piece of `tile` are consecutive: [first, first + count). Only the first one can
// have started in an earlier tile (its piece of this tile is its segment `seg_first`); the others start inside the
// tile, so their piece is their segment 0. Every span is non-empty because ctas <= units_total.
__device__ __forceinline__ void q80_tile_ctas(const Q80EpiArgs& e, uint32_t tile, uint32_t* first, uint32_t* count,
                                              uint32_t* seg_first) {
    const uint32_t t0 = tile * e.units_per_tile, t1 = t0 + e.units_per_tile;
    uint32_t c = (t0 * e.ctas) / e.units_total;
    while (((c + 1u) * e.units_total) / e.ctas <= t0) ++c;
    *first = c;
    *seg_first = tile - ((c * e.units_total) / e.ctas) / e.units_per_tile;
    uint32_t n = 0;
    while (c < e.ctas && (c * e.units_total) / e.ctas < t1) {
        ++c;
        ++n;
    }
    *count = n;
}

// grid (tiles of the widest problem, ceil(M / 8), problems or 1), block 256: thread = (tile row, lane of 2) walking
// 8 activation rows.
__global__ void __launch_bounds__(256) gemm_tc_q80_epilogue_kernel(Q80EpiArgs e) {
    __shared__ uint32_t first[2], count[2], seg0[2];
    const uint32_t p = blockIdx.z, t = blockIdx.x, tr = threadIdx.x & 127u;
    const uint32_t n = t * BLOCK_N + tr;
    // which CTAs hold this tile follows from the launch arguments alone: worked out while the GEMM still runs
    if (t * BLOCK_N < e.N[p]) {
        if (threadIdx.x == 0) q80_tile_ctas(e, e.tile_begin[p] + t, &first[0], &count[0], &seg0[0]);
        if (threadIdx.x == 32 && e.mode == 1) q80_tile_ctas(e, e.tile_begin[1] + t, &first[1], &count[1], &seg0[1]);
    }
    pdl_wait();
    pdl_trigger();
    if (t * BLOCK_N >= e.N[p]) return;
    __syncthreads();
    if (n >= e.N[p]) return;
    // A thread owns 4 activation rows. Every load of a round is unconditional (row and partial index clamped, the value
    // masked afterwards) and issued before any is added: guarded loads were issued one at a time, each waiting for
    // the previous one's trip to L2. The adds keep a fixed order.
    const uint32_t m0 = blockIdx.y * 8u + (threadIdx.x >> 7);
    const uint32_t M = e.M, seg_max = e.seg_max;
    const float* __restrict__ part = e.partial + tr;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint32_t c0 = count[0], c1 = e.mode == 1 ? count[1] : 0u;
    const uint32_t cmax = c0 > c1 ? c0 : c1;
    for (uint32_t i0 = 0; i0 < cmax; i0 += 4u) {
        float v[2][4][4];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            const uint32_t cw = w == 0 ? c0 : c1;
            if (w == 1 && c1 == 0u) break;
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t m = min(m0 + 2u * r, M - 1u), i = min(i0 + k, cw - 1u);
                    const size_t slot = (size_t)(first[w] + i) * seg_max + (i == 0 ? seg0[w] : 0u);
                    v[w][r][k] = part[(slot * M + m) * BLOCK_N];
                }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc[r] += (i0 + k < c0) ? v[0][r][k] : 0.0f;
                if (c1 != 0u) up[r] += (i0 + k < c1) ? v[1][r][k] : 0.0f;
            }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t m = m0 + 2u * r;
        if (m >= e.M) continue;
        float a0 = acc[r];
        if (e.mode == 1) {
            const float v = (a0 / (1.0f + expf(-a0))) * up[r];
            const size_t o = (size_t)m * e.N[0] + n;
            e.out[0][o] = v;
            if (e.split_hi) {  // the same split as split_activations_kernel
                const __half h = __float2half_rn(v);
                e.split_hi[o] = h;
                e.split_lo[o] = __float2half_rn(v - __half2float(h));
            }
            continue;
        }
        if (e.residual[p]) a0 += e.residual[p][(size_t)m * e.N[p] + n];
        e.out[p][(size_t)m * e.N[p] + n] = a0;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

bool make_map_raw(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return false;
    const cuuint64_t dims[2] = {row_bytes / 2, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {RAW_ROW_BYTES / 2, BLOCK_N};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_map_act(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {BLOCK_K, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int M_PAD>
int launch_q80(M40llmCudaContext* ctx, cudaStream_t s, const CUtensorMap* mW, const CUtensorMap& mXh,
               const CUtensorMap& mXl, const Q80Args& a) {
    constexpr size_t smem = RS * RAW_BYTES + b_slots(M_PAD) * 2 * (M_PAD * BLOCK_K * 2) + 64 * 8 + 16 + 1024;
    auto kern = gemm_tc_q80_kernel<M_PAD>;
    static unsigned long long configured = 0ull;
    const unsigned long long bit = 1ull << (ctx->device_id & 63);
    if (!(configured & bit)) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -2;
        configured |= bit;
    }
    m40_launch_dependent(kern, dim3(a.ctas), dim3(CTA_THREADS), smem, s, mW[0], mW[1], mW[2], mXh, mXl, a);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace

bool m40_gemm_tc_q80_supported(int M, int K, int problems, const void* const* W) {
    if (M < 2 || M > 64 || K % 256 != 0 || problems < 1 || problems > 3) return false;
    for (int p = 0; p < problems; ++p)
        if ((((uintptr_t)W[p]) & 15u) != 0u) return false;
    return get_encode() != nullptr;
}

namespace {
// Tile / span bookkeeping shared by the launch and the scratch query.
void q80_plan(const M40llmCudaContext* ctx, int M, int K, int problems, const int* N, Q80Args* a) {
    a->M = (uint32_t)M;
    a->K = (uint32_t)K;
    a->problems = (uint32_t)problems;
    uint32_t tiles = 0;
    for (int p = 0; p < problems; ++p) {
        a->tile_begin[p] = tiles;
        tiles += (uint32_t)((N[p] + BLOCK_N - 1) / BLOCK_N);
    }
    for (int p = problems; p < 4; ++p) a->tile_begin[p] = tiles;
    a->tiles_total = tiles;
    a->units_per_tile = (uint32_t)K / UNIT_K;
    a->units_total = tiles * a->units_per_tile;
    a->ctas = (uint32_t)ctx->sm_count < a->units_total ? (uint32_t)ctx->sm_count : a->units_total;
    const uint32_t upc = (a->units_total + a->ctas - 1) / a->ctas;
    a->seg_max = upc / a->units_per_tile + 2;
}
size_t q80_act_bytes(int M, int K) { return (((size_t)M * K * 2 + 255) / 256) * 256; }
}  // namespace

void m40_gemm_tc_q80_scratch(const M40llmCudaContext* ctx, int M, int K, int problems, const int* N, size_t* act_bytes,
                             size_t* part_bytes) {
    Q80Args a = {};
    q80_plan(ctx, M, K, problems, N, &a);
    *act_bytes = q80_act_bytes(M, K);
    *part_bytes = (size_t)a.ctas * a.seg_max * M * BLOCK_N * sizeof(float);
}

int m40_gemm_tc_q80(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* X, int M, int K,
                    int problems, const uint8_t* const* W, const int* N, float* const* out,
                    const float* const* residual, int mode, const M40GemvNorm* norm, const M40TcChain* chain) {
    const uint32_t M_pad = M <= 16 ? 16u : (M <= 32 ? 32u : 64u);
    Q80Args a = {};
    q80_plan(ctx, M, K, problems, N, &a);
    if ((uint64_t)(a.units_total + 1) * (a.ctas + 1) >= (1ull << 32)) return -2;  // span arithmetic is 32-bit

    const size_t act_bytes = q80_act_bytes(M, K);
    const size_t part_bytes = (size_t)a.ctas * a.seg_max * M * BLOCK_N * sizeof(float);
    size_t need = 2 * act_bytes + part_bytes;
    if (chain && chain->scratch_bytes > need) need = chain->scratch_bytes;
    unsigned char* scratch = (unsigned char*)m40_ensure_scratch(ctx, stream_kind, need);
    if (!scratch) return -2;
    const bool presplit = chain && chain->read_split;
    // own split copies in front of the partial tiles; with pre-split activations the partial tiles come first
    __half* xh = (__half*)(presplit ? scratch + chain->act_off : scratch);
    __half* xl = (__half*)((unsigned char*)xh + act_bytes);
    a.partial = (float*)(presplit ? scratch : scratch + 2 * act_bytes);
    a.status = ctx->d_status;

    const uint64_t row_bytes = (uint64_t)(K / 32) * 34;
    CUtensorMap mW[3], mXh, mXl;
    for (int p = 0; p < 3; ++p) {
        const int q = p < problems ? p : 0;
        if (!make_map_raw(&mW[p], W[q], (uint64_t)N[q], row_bytes)) return -2;
    }
    if (!make_map_act(&mXh, xh, (uint64_t)M, (uint64_t)K, M_pad)) return -2;
    if (!make_map_act(&mXl, xl, (uint64_t)M, (uint64_t)K, M_pad)) return -2;
    if (!presplit && m40_split_activations(ctx, s, X, xh, xl, M, K, norm) != 0) return -2;
    int rc;
    if (M_pad == 16) rc = launch_q80<16>(ctx, s, mW, mXh, mXl, a);
    else if (M_pad == 32) rc = launch_q80<32>(ctx, s, mW, mXh, mXl, a);
    else rc = launch_q80<64>(ctx, s, mW, mXh, mXl, a);
    if (rc != 0) return rc;

    Q80EpiArgs e = {};
    e.partial = a.partial;
    if (chain && chain->write_split && mode == 1) {
        e.split_hi = (__half*)(scratch + chain->act_off);
        e.split_lo = (__half*)(scratch + chain->act_off + q80_act_bytes(M, N[0]));
    }
    uint32_t maxN = 0;
    for (int p = 0; p < problems; ++p) {
        e.out[p] = out[p];
        e.residual[p] = residual ? residual[p] : nullptr;
        e.N[p] = (uint32_t)N[p];
        if ((uint32_t)N[p] > maxN) maxN = (uint32_t)N[p];
    }
    for (int p = 0; p < 4; ++p) e.tile_begin[p] = a.tile_begin[p];
    e.M = (uint32_t)M;
    e.units_per_tile = a.units_per_tile;
    e.units_total = a.units_total;
    e.ctas = a.ctas;
    e.seg_max = a.seg_max;
    e.mode = (uint32_t)mode;
    e.problems = (uint32_t)problems;
    dim3 egrid((maxN + BLOCK_N - 1) / BLOCK_N, (unsigned)(M + 7) / 8, mode == 1 ? 1u : (unsigned)problems);
    m40_launch_dependent(gemm_tc_q80_epilogue_kernel, egrid, dim3(256), 0, s, e);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
