// Batched decode projections over Q8_0 GGUF rows on the tcgen05 tensor cores.
//
// Q8_0 stores 32 weights as {f16 d; int8 q[32]} (34 bytes, cuda/kernels.cu:856-867 of the reference):
// w = d * q with a different d for every (row, 32-k block). The kernel keeps that structure exact:
//
//   raw bytes   TMA (plain 2D box of 128 rows x 272 bytes = 8 blocks per row) straight from the GGUF layout;
//   int8 -> f16 worker threads (one weight row each) turn q into exact f16 integers and write them into the
//               128-byte-swizzled K-major tile the MMA reads; d stays in a register;
//   MMA         per 32-k block a FRESH accumulator D_b[128 x M_pad] = Q_b . Xt_b in TMEM (activations as f16
//               hi + lo parts, so D_b is exact to f32 rounding); four TMEM buffers rotate;
//   scale       the same worker threads read their row of D_b back (tcgen05.ld) and do
//               acc[m] += d * D_b[m] in f32 registers  -- the reference's d*q product, just re-associated.
//
// Work is split stream-K style: the (tile, 256-k unit) space is cut into one contiguous span per CTA
// (one CTA per SM; shared memory holds two raw stages + rings), so every SM streams the same number of
// weight bytes. A span that crosses tile boundaries writes one partial per tile; the epilogue kernel adds
// the partials of each tile and applies residual or SiLU(gate)*up.
//
// Every wait is bounded; a wait that runs out sets bit 2 of the context's device status word and the CTA
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
constexpr uint32_t A_BYTES = BLOCK_N * BLOCK_K * 2;    // 16384: one converted 64-k sub-block
constexpr uint32_t RS = 2, AS = 2, BS = 4, TB = 4;     // ring depths: raw stages, A slots, B slots, TMEM buffers

struct Q80Args {
    float* partial;  // [ctas][seg_max][M][128]
    uint32_t* status;
    uint32_t M, K;
    uint32_t tile_begin[4], problems, tiles_total;
    uint32_t units_per_tile;  // K / 256
    uint32_t units_total, ctas, seg_max;
};

__device__ __forceinline__ void span_of(const Q80Args& a, uint32_t cta, uint32_t* u0, uint32_t* u1) {
    *u0 = (uint32_t)(((uint64_t)cta * a.units_total) / a.ctas);
    *u1 = (uint32_t)(((uint64_t)(cta + 1) * a.units_total) / a.ctas);
}

template <int M_PAD>
__global__ void __launch_bounds__(192, 1) gemm_tc_q80_kernel(const __grid_constant__ CUtensorMap tmW0,
                                                             const __grid_constant__ CUtensorMap tmW1,
                                                             const __grid_constant__ CUtensorMap tmW2,
                                                             const __grid_constant__ CUtensorMap tmXh,
                                                             const __grid_constant__ CUtensorMap tmXl, Q80Args a) {
    constexpr uint32_t B_BYTES = M_PAD * BLOCK_K * 2;  // one of hi / lo for a 64-k sub-block
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    unsigned char* s_raw = smem;                             // RS x RAW_BYTES
    unsigned char* s_a = s_raw + RS * RAW_BYTES;             // AS x A_BYTES (1024-aligned: RAW_BYTES = 34 * 1024)
    unsigned char* s_b = s_a + AS * A_BYTES;                 // BS x (hi, lo)
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_b + BS * 2 * B_BYTES);
    uint64_t* raw_full = bars;
    uint64_t* raw_empty = raw_full + RS;
    uint64_t* a_full = raw_empty + RS;
    uint64_t* a_empty = a_full + AS;
    uint64_t* b_full = a_empty + AS;
    uint64_t* b_empty = b_full + BS;
    uint64_t* t_full = b_empty + BS;
    uint64_t* t_empty = t_full + TB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(t_empty + TB);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    constexpr uint32_t TMEM_COLS = TB * M_PAD < 32 ? 32 : TB * M_PAD;  // 64 / 128 / 256: powers of two

    uint32_t u0, u1;
    span_of(a, blockIdx.x, &u0, &u1);
    const uint32_t n_units = u1 - u0;

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < RS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 128); }
        for (uint32_t i = 0; i < AS; ++i) { mbar_init(&a_full[i], 128); mbar_init(&a_empty[i], 1); }
        for (uint32_t i = 0; i < BS; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
        for (uint32_t i = 0; i < TB; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer
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
                for (uint32_t sub = 0; sub < 4; ++sub) {
                    const uint32_t u = i * 4 + sub, bs = u % BS;
                    if (u >= BS && !mbar_wait(&b_empty[bs], ((u / BS) - 1) & 1u)) { ok = false; break; }
                    mbar_expect_tx(&b_full[bs], 2 * B_BYTES);
                    const int kx = (int)(kb * UNIT_K + sub * BLOCK_K);
                    tma_load_2d(s_b + bs * 2 * B_BYTES, &tmXh, &b_full[bs], kx, 0);
                    tma_load_2d(s_b + bs * 2 * B_BYTES + B_BYTES, &tmXl, &b_full[bs], kx, 0);
                }
            }
            if (!ok) *abort_flag = 1;
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: per 32-k block a fresh accumulator in TMEM buffer v % TB
        if (lane == 0) {
            const uint32_t idesc = make_idesc(M_PAD);
            bool ok = true;
            for (uint32_t u = 0; u < n_units * 4 && ok; ++u) {
                const uint32_t as = u % AS, bs = u % BS;
                if (!mbar_wait(&a_full[as], (u / AS) & 1u) || !mbar_wait(&b_full[bs], (u / BS) & 1u)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sa = smem_u32(s_a + as * A_BYTES);
                const uint32_t sb = smem_u32(s_b + bs * 2 * B_BYTES);
                for (uint32_t blk = 0; blk < 2 && ok; ++blk) {
                    const uint32_t v = u * 2 + blk, tb = v % TB;
                    if (v >= TB && !mbar_wait(&t_empty[tb], ((v / TB) - 1) & 1u)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + tb * M_PAD;
#pragma unroll
                    for (uint32_t kk = 0; kk < 2; ++kk) {
                        const uint32_t off = (blk * 2 + kk) * UMMA_K * 2;
                        const uint64_t da = make_desc_sw128(sa + off);
                        umma_f16(d_tmem, da, make_desc_sw128(sb + off), idesc, kk);
                        umma_f16(d_tmem, da, make_desc_sw128(sb + B_BYTES + off), idesc, 1u);
                    }
                    umma_commit(&t_full[tb]);
                }
                if (ok) {
                    umma_commit(&a_empty[as]);
                    umma_commit(&b_empty[bs]);
                }
            }
            if (!ok) *abort_flag = 1;
        }
    } else {
        // ---------------- workers: convert int8 -> f16 tiles, then scale-accumulate the block results
        const uint32_t lane_group = warp & 3u;
        const uint32_t r = lane_group * 32 + lane;  // weight row of the tile == TMEM lane
        float acc[M_PAD];
        float d_prev0 = 0.f, d_prev1 = 0.f;
        bool ok = true;
        uint32_t ucount = 0;  // sub-blocks handled so far by this CTA
        // every wait of a worker warp is made warp-uniform so the warp-collective tcgen05.ld stays converged
        auto wwait = [&](uint64_t* bar, uint32_t parity) {
            const bool r0 = mbar_wait(bar, parity);
            return (bool)__all_sync(0xffffffffu, r0);
        };

        auto accumulate = [&](uint32_t u, float d0, float d1) {
#pragma unroll
            for (uint32_t blk = 0; blk < 2; ++blk) {
                const uint32_t v = u * 2 + blk, tb = v % TB;
                if (!wwait(&t_full[tb], (v / TB) & 1u)) {
                    ok = false;
                    return;
                }
                tc_fence_after();
                const float d = blk == 0 ? d0 : d1;
#pragma unroll
                for (uint32_t c = 0; c < M_PAD; c += 8) {
                    float x[8];
                    tmem_ld8(tmem_base + ((lane_group * 32u) << 16) + tb * M_PAD + c, x);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[c + j] = fmaf(d, x[j], acc[c + j]);
                }
                tc_fence_before();
                mbar_arrive(&t_empty[tb]);
            }
        };

        uint32_t pos = u0, seg = 0;
        while (pos < u1 && ok) {
            const uint32_t tile = pos / a.units_per_tile;
            const uint32_t kb_begin = pos % a.units_per_tile;
            uint32_t kb_end = kb_begin + (u1 - pos);
            if (kb_end > a.units_per_tile) kb_end = a.units_per_tile;
#pragma unroll
            for (int m = 0; m < M_PAD; ++m) acc[m] = 0.0f;
            const uint32_t seg_first = ucount;
            for (uint32_t kb = kb_begin; kb < kb_end && ok; ++kb) {
                const uint32_t i = ucount / 4, rs = i % RS;
                if (!wwait(&raw_full[rs], (i / RS) & 1u)) { ok = false; break; }
                const uint4* raw = reinterpret_cast<const uint4*>(s_raw + rs * RAW_BYTES + r * RAW_ROW_BYTES);
#pragma unroll
                for (uint32_t sub = 0; sub < 4; ++sub) {
                    const uint32_t u = ucount, as = u % AS;
                    if (u >= AS && !wwait(&a_empty[as], ((u / AS) - 1) & 1u)) { ok = false; break; }
                    // 68 bytes of this row: {d0, q0[32], d1, q1[32]} = words W[0..16], starting at word 17*sub
                    uint32_t buf[20];
#pragma unroll
                    for (int c = 0; c < 5; ++c) {
                        const uint4 t = raw[4 * sub + c];
                        buf[4 * c] = t.x; buf[4 * c + 1] = t.y; buf[4 * c + 2] = t.z; buf[4 * c + 3] = t.w;
                    }
                    const uint32_t* W = buf + sub;
                    const float d0 = __half2float(__ushort_as_half((unsigned short)(W[0] & 0xffffu)));
                    const float d1 = __half2float(__ushort_as_half((unsigned short)(W[8] >> 16)));
                    unsigned char* dst = s_a + as * A_BYTES + (r >> 3) * 1024 + (r & 7u) * 128;
                    const __half2 bias = __float2half2_rn(1152.0f);
#pragma unroll
                    for (uint32_t c = 0; c < 8; ++c) {
                        uint32_t o[4];
#pragma unroll
                        for (uint32_t pp = 0; pp < 4; ++pp) {
                            const uint32_t p = (c & 3u) * 4 + pp;  // pair index inside its Q8_0 block
                            uint32_t word, upper;
                            if (c < 4) { word = W[(p + 1) >> 1]; upper = (p & 1u) == 0u; }   // block 0: bytes 2 + 2p
                            else { word = W[9 + (p >> 1)]; upper = (p & 1u) == 1u; }           // block 1: bytes 36 + 2p
                            const uint32_t x = word ^ 0x80808080u;
                            const uint32_t h = __byte_perm(x, 0x64646464u, upper ? 0x7362 : 0x5140);  // (1024+u0, 1024+u1)
                            const __half2 q2 = __hsub2(*reinterpret_cast<const __half2*>(&h), bias);   // exact ints
                            o[pp] = *reinterpret_cast<const uint32_t*>(&q2);
                        }
                        *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7u)) * 16)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(&a_full[as]);
                    if (u > seg_first) accumulate(u - 1, d_prev0, d_prev1);
                    if (!ok) break;
                    d_prev0 = d0;
                    d_prev1 = d1;
                    ++ucount;
                }
                if (!ok) break;
                mbar_arrive(&raw_empty[rs]);
            }
            if (ok && ucount > seg_first) accumulate(ucount - 1, d_prev0, d_prev1);
            if (ok) {
                float* dst = a.partial + ((size_t)(blockIdx.x * a.seg_max + seg) * a.M) * BLOCK_N + r;
#pragma unroll
                for (int m = 0; m < M_PAD; ++m)
                    if ((uint32_t)m < a.M) dst[(size_t)m * BLOCK_N] = acc[m];
            }
            (void)tile;
            pos += kb_end - kb_begin;
            ++seg;
        }
        if (!ok) *abort_flag = 1;
    }
    if (*abort_flag && threadIdx.x == 64) atomicOr(a.status, 4u);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

struct Q80EpiArgs {
    const float* partial;
    float* out[3];
    const float* residual[3];
    uint32_t N[3];
    uint32_t tile_begin[4];
    uint32_t M, units_per_tile, units_total, ctas, seg_max, mode;
};

__device__ __forceinline__ float q80_tile_sum(const Q80EpiArgs& e, uint32_t tile, uint32_t m, uint32_t n_local) {
    const uint32_t t0 = tile * e.units_per_tile, t1 = t0 + e.units_per_tile;
    // first CTA whose span reaches into this tile
    uint32_t c = (uint32_t)(((uint64_t)t0 * e.ctas) / e.units_total);
    while (c > 0 && (uint32_t)(((uint64_t)c * e.units_total) / e.ctas) > t0) --c;
    while ((uint32_t)(((uint64_t)(c + 1) * e.units_total) / e.ctas) <= t0) ++c;
    float acc = 0.0f;
    for (; c < e.ctas; ++c) {
        const uint32_t u0 = (uint32_t)(((uint64_t)c * e.units_total) / e.ctas);
        const uint32_t u1 = (uint32_t)(((uint64_t)(c + 1) * e.units_total) / e.ctas);
        if (u0 >= t1) break;
        if (u1 <= t0 || u1 == u0) continue;
        const uint32_t seg = tile - u0 / e.units_per_tile;  // this tile's position among the CTA's tiles
        acc += e.partial[((size_t)(c * e.seg_max + seg) * e.M + m) * BLOCK_N + n_local];
    }
    return acc;
}

__global__ void gemm_tc_q80_epilogue_kernel(Q80EpiArgs e) {
    const uint32_t p = blockIdx.z, m = blockIdx.y;
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= e.N[p]) return;
    float acc = q80_tile_sum(e, e.tile_begin[p] + n / BLOCK_N, m, n % BLOCK_N);
    if (e.mode == 1) {
        const float up = q80_tile_sum(e, e.tile_begin[1] + n / BLOCK_N, m, n % BLOCK_N);
        e.out[0][(size_t)m * e.N[0] + n] = (acc / (1.0f + expf(-acc))) * up;
        return;
    }
    if (e.residual[p]) acc += e.residual[p][(size_t)m * e.N[p] + n];
    e.out[p][(size_t)m * e.N[p] + n] = acc;
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

__global__ void split_activations_q80_kernel(const float* __restrict__ x, __half* __restrict__ hi,
                                             __half* __restrict__ lo, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = x[i];
        const __half h = __float2half_rn(v);
        hi[i] = h;
        lo[i] = __float2half_rn(v - __half2float(h));
    }
}

template <int M_PAD>
int launch_q80(M40llmCudaContext* ctx, cudaStream_t s, const CUtensorMap* mW, const CUtensorMap& mXh,
               const CUtensorMap& mXl, const Q80Args& a) {
    constexpr size_t smem = RS * RAW_BYTES + AS * A_BYTES + BS * 2 * (M_PAD * BLOCK_K * 2) + 32 * 8 + 16 + 1024;
    auto kern = gemm_tc_q80_kernel<M_PAD>;
    static unsigned long long configured = 0ull;
    const unsigned long long bit = 1ull << (ctx->device_id & 63);
    if (!(configured & bit)) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -2;
        configured |= bit;
    }
    kern<<<a.ctas, 192, smem, s>>>(mW[0], mW[1], mW[2], mXh, mXl, a);
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

int m40_gemm_tc_q80(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* X, int M, int K,
                    int problems, const uint8_t* const* W, const int* N, float* const* out,
                    const float* const* residual, int mode) {
    const uint32_t M_pad = M <= 16 ? 16u : (M <= 32 ? 32u : 64u);
    Q80Args a = {};
    a.M = (uint32_t)M;
    a.K = (uint32_t)K;
    a.problems = (uint32_t)problems;
    uint32_t tiles = 0;
    for (int p = 0; p < problems; ++p) {
        a.tile_begin[p] = tiles;
        tiles += (uint32_t)((N[p] + BLOCK_N - 1) / BLOCK_N);
    }
    for (int p = problems; p < 4; ++p) a.tile_begin[p] = tiles;
    a.tiles_total = tiles;
    a.units_per_tile = (uint32_t)K / UNIT_K;
    a.units_total = tiles * a.units_per_tile;
    a.ctas = (uint32_t)ctx->sm_count < a.units_total ? (uint32_t)ctx->sm_count : a.units_total;
    const uint32_t upc = (a.units_total + a.ctas - 1) / a.ctas;
    a.seg_max = upc / a.units_per_tile + 2;

    const size_t act_elems = (size_t)M * K;
    const size_t act_bytes = ((act_elems * 2 + 255) / 256) * 256;
    const size_t part_bytes = (size_t)a.ctas * a.seg_max * M * BLOCK_N * sizeof(float);
    unsigned char* scratch = (unsigned char*)m40_ensure_scratch(ctx, stream_kind, 2 * act_bytes + part_bytes);
    if (!scratch) return -2;
    __half* xh = (__half*)scratch;
    __half* xl = (__half*)(scratch + act_bytes);
    a.partial = (float*)(scratch + 2 * act_bytes);
    a.status = ctx->d_status;

    const uint64_t row_bytes = (uint64_t)(K / 32) * 34;
    CUtensorMap mW[3], mXh, mXl;
    for (int p = 0; p < 3; ++p) {
        const int q = p < problems ? p : 0;
        if (!make_map_raw(&mW[p], W[q], (uint64_t)N[q], row_bytes)) return -2;
    }
    if (!make_map_act(&mXh, xh, (uint64_t)M, (uint64_t)K, M_pad)) return -2;
    if (!make_map_act(&mXl, xl, (uint64_t)M, (uint64_t)K, M_pad)) return -2;
    {
        size_t blocks = (act_elems + 255) / 256;
        if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
        split_activations_q80_kernel<<<(unsigned)blocks, 256, 0, s>>>(X, xh, xl, act_elems);
        M40_COUNT_LAUNCH(ctx);
    }
    int rc;
    if (M_pad == 16) rc = launch_q80<16>(ctx, s, mW, mXh, mXl, a);
    else if (M_pad == 32) rc = launch_q80<32>(ctx, s, mW, mXh, mXl, a);
    else rc = launch_q80<64>(ctx, s, mW, mXh, mXl, a);
    if (rc != 0) return rc;

    Q80EpiArgs e = {};
    e.partial = a.partial;
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
    dim3 egrid((maxN + 255) / 256, (unsigned)M, mode == 1 ? 1u : (unsigned)problems);
    gemm_tc_q80_epilogue_kernel<<<egrid, 256, 0, s>>>(e);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
