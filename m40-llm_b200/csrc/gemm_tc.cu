// Batched decode projections on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// For M >= 2 activation rows the projection C[m][n] = sum_k X[m][k] W[n][k] is computed "swapped":
// the streamed weight tile is the MMA's A operand (128 weight rows = the MMA M dimension) and the
// small activation matrix is the B operand (MMA N = batch rows padded to 16..256), so the tensor core
// runs at full height however small the batch is and every weight byte is read from HBM exactly once:
//
//   D[n_tile 128 x M_pad] (f32, in TMEM)  +=  W[128 x 64] (f16, smem, TMA 128B-swizzled)
//                                            * Xt[64 x M_pad] (f16, smem, TMA 128B-swizzled)
//
// f32 activations are split into f16 hi + lo parts (two MMAs per k-step; tensor time is free while the
// kernel is HBM-bound), so results keep f32-level accuracy for small batches.
//
// Roles inside a CTA (6 warps): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
// epilogue (TMEM -> registers -> global partials). Up to three weight matrices that share the
// activations (Wq|Wk|Wv, Wgate|Wup) are one launch; K is split over grid.y so that about two CTAs per
// SM are resident. Partials land in scratch and a small second kernel adds the K splits and applies the
// epilogue (bias, residual, or SiLU(gate)*up).
//
// Every wait is bounded: a wait that runs out sets bit 2 of the context's device status word, the
// CTA stops issuing work, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace {

using namespace tc;

struct TcArgs {
    float* partial;            // [k_splits][M][n_total]
    uint32_t* status;
    uint32_t M, M_pad, K;
    uint32_t n_total;          // sum of padded tile rows over the problems (n_tiles_total * 128)
    uint32_t tile_begin[4];    // first tile of each problem, tile_begin[problems] = total
    uint32_t problems;
    uint32_t kblocks_per_split, kblocks_total;
    uint32_t use_lo;           // 1: activations carry a lo part (second MMA)
    uint32_t stages;
};

__global__ void __launch_bounds__(192, 1) gemm_tc_f16_kernel(const __grid_constant__ CUtensorMap tmW0,
                                                             const __grid_constant__ CUtensorMap tmW1,
                                                             const __grid_constant__ CUtensorMap tmW2,
                                                             const __grid_constant__ CUtensorMap tmXh,
                                                             const __grid_constant__ CUtensorMap tmXl, TcArgs a) {
    extern __shared__ unsigned char smem_unaligned[];
    // the swizzled tiles must start on 1024-byte boundaries; the launch reserves the slack
    unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tile = blockIdx.x, ksplit = blockIdx.y;
    const uint32_t a_bytes = BLOCK_N * BLOCK_K * 2;                 // 16 KB
    const uint32_t b_bytes = a.M_pad * BLOCK_K * 2;                 // per hi / lo part
    const uint32_t stage_bytes = a_bytes + (a.use_lo ? 2u : 1u) * b_bytes;
    unsigned char* stage_base = smem;                                // stages * stage_bytes, 1024-aligned each
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + a.stages * stage_bytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + a.stages;
    uint64_t* accum = bars + 2 * a.stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * a.stages + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    // hi and lo activation tiles are contiguous rows of one operand: up to M_pad = 128 a single MMA of width
    // 2 * M_pad takes the weight tile against both (the weight operand passes the tensor core once); the two
    // halves of the accumulator are added in the epilogue.
    const bool stacked = a.use_lo && a.M_pad <= 128u;
    const uint32_t acc_cols = stacked ? 2u * a.M_pad : a.M_pad;
    uint32_t tmem_cols = 32;
    while (tmem_cols < acc_cols) tmem_cols <<= 1;

    uint32_t problem = 0;
    while (problem + 1 < a.problems && tile >= a.tile_begin[problem + 1]) ++problem;
    const CUtensorMap* tmW = problem == 0 ? &tmW0 : (problem == 1 ? &tmW1 : &tmW2);
    const uint32_t row0 = (tile - a.tile_begin[problem]) * BLOCK_N;
    const uint32_t kb0 = ksplit * a.kblocks_per_split;
    uint32_t kb1 = kb0 + a.kblocks_per_split;
    if (kb1 > a.kblocks_total) kb1 = a.kblocks_total;
    const uint32_t n_kb = kb1 > kb0 ? kb1 - kb0 : 0u;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer. The weight tiles of the first ring pass do not depend on the previous kernel:
        // they are requested before the dependency wait, the activation tiles after it.
        if (lane == 0) {
            const uint32_t pre = n_kb < a.stages ? n_kb : a.stages;
            for (uint32_t i = 0; i < pre; ++i) {
                mbar_expect_tx(&full[i], stage_bytes);
                tma_load_2d(stage_base + i * stage_bytes, tmW, &full[i], (int)((kb0 + i) * BLOCK_K), (int)row0);
            }
            pdl_wait();
            for (uint32_t i = 0; i < pre; ++i) {
                unsigned char* st = stage_base + i * stage_bytes;
                const int kx = (int)((kb0 + i) * BLOCK_K);
                tma_load_2d(st + a_bytes, &tmXh, &full[i], kx, 0);
                if (a.use_lo) tma_load_2d(st + a_bytes + b_bytes, &tmXl, &full[i], kx, 0);
            }
            for (uint32_t i = pre; i < n_kb; ++i) {
                const uint32_t s = i % a.stages, round = i / a.stages;
                if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1u)) { *abort_flag = 1; break; }
                if (*abort_flag) break;
                unsigned char* st = stage_base + s * stage_bytes;
                mbar_expect_tx(&full[s], stage_bytes);
                const int kx = (int)((kb0 + i) * BLOCK_K);
                tma_load_2d(st, tmW, &full[s], kx, (int)row0);
                tma_load_2d(st + a_bytes, &tmXh, &full[s], kx, 0);
                if (a.use_lo) tma_load_2d(st + a_bytes + b_bytes, &tmXl, &full[s], kx, 0);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc(acc_cols);
            bool ok = true;
            for (uint32_t i = 0; i < n_kb && ok; ++i) {
                const uint32_t s = i % a.stages, round = i / a.stages;
                if (!mbar_wait(&full[s], round & 1u)) { *abort_flag = 1; ok = false; break; }
                tc_fence_after();
                const uint32_t sa = smem_u32(stage_base + s * stage_bytes);
                const uint32_t sb = sa + a_bytes;
#pragma unroll
                for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t da = make_desc_sw128(sa + k * UMMA_K * 2);
                    umma_f16(tmem_base, da, make_desc_sw128(sb + k * UMMA_K * 2), idesc, (i | k) != 0u);
                    if (a.use_lo && !stacked) umma_f16(tmem_base, da, make_desc_sw128(sb + b_bytes + k * UMMA_K * 2), idesc, 1u);
                }
                umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(accum);  // accumulator complete
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lanes 32*(warp % 4) .. +31
        const uint32_t lane_group = warp & 3u;
        pdl_wait();  // the partials below reuse scratch that earlier kernels may still read
        bool ok = n_kb > 0;
        if (ok) {
            if (!mbar_wait(accum, 0)) { *abort_flag = 1; ok = false; }
        }
        ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective
        tc_fence_after();
        const uint32_t n_glob = tile * BLOCK_N + lane_group * 32 + lane;
        float* dst = a.partial + (size_t)ksplit * a.M * a.n_total + n_glob;
        for (uint32_t c = 0; c < a.M_pad; c += 8) {
            float v[8];
            if (ok) {
                tmem_ld8(tmem_base + ((lane_group * 32u) << 16) + c, v);
                if (stacked) {
                    float w[8];
                    tmem_ld8(tmem_base + ((lane_group * 32u) << 16) + a.M_pad + c, w);
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] += w[j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (c + j < a.M) dst[(size_t)(c + j) * a.n_total] = v[j];
        }
    }
    if (*abort_flag && threadIdx.x == 64) atomicOr(a.status, 4u);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// f32 activations -> f16 hi (+ lo) copies, [M][K] row-major.
__global__ void split_activations_kernel(const float* __restrict__ x, __half* __restrict__ hi, __half* __restrict__ lo,
                                         size_t n) {
    pdl_wait();
    pdl_trigger();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = x[i];
        const __half h = __float2half_rn(v);
        hi[i] = h;
        if (lo) lo[i] = __float2half_rn(v - __half2float(h));
    }
}

// One CTA per activation row: RMSNorm (x * rsqrt(mean(x^2) + eps) * w), then the f16 hi/lo split. The row and its
// norm weights are fetched once, all loads in flight together (up to 8192 columns stay in registers; wider rows are
// read a second time for the part beyond).
// w_f32: bit 0 = f32 weights (else f16), bit 1 = the weight pointer is not aligned for vector loads
__device__ __forceinline__ float4 norm_w4(const void* w, int w_f32, uint32_t k) {
    if (w_f32 & 2) {
        float t[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            t[i] = (w_f32 & 1) ? reinterpret_cast<const float*>(w)[k + i]
                               : __half2float(reinterpret_cast<const __half*>(w)[k + i]);
        return make_float4(t[0], t[1], t[2], t[3]);
    }
    if (w_f32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + k);
    const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(w) + k);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void split_store4(const float4& x, const float4& wv, float scale, __half* hr, __half* lr) {
    const float y[4] = {x.x * scale * wv.x, x.y * scale * wv.y, x.z * scale * wv.z, x.w * scale * wv.w};
    __half h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h[i] = __float2half_rn(y[i]);
        l[i] = __float2half_rn(y[i] - __half2float(h[i]));
    }
    *reinterpret_cast<uint2*>(hr) = *reinterpret_cast<const uint2*>(h);
    *reinterpret_cast<uint2*>(lr) = *reinterpret_cast<const uint2*>(l);
}
__global__ void __launch_bounds__(256) norm_split_rows_kernel(const float* __restrict__ x, const void* __restrict__ w,
                                                              int w_f32, float eps, __half* __restrict__ hi,
                                                              __half* __restrict__ lo, uint32_t K) {
    __shared__ float red[8];
    pdl_wait();
    pdl_trigger();
    const float* xr = x + (size_t)blockIdx.x * K;
    __half* hr = hi + (size_t)blockIdx.x * K;
    __half* lr = lo + (size_t)blockIdx.x * K;
    constexpr int V = 8;  // float4 per thread held in registers
    float4 xv[V], wv[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const uint32_t k = threadIdx.x * 4u + (uint32_t)i * 1024u;
        xv[i] = k < K ? *reinterpret_cast<const float4*>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        wv[i] = k < K ? norm_w4(w, w_f32, k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) ss += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
    for (uint32_t k = threadIdx.x * 4u + V * 1024u; k < K; k += 1024u) {
        const float4 v = *reinterpret_cast<const float4*>(xr + k);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0u) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float scale = rsqrtf(tot / (float)K + eps);
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const uint32_t k = threadIdx.x * 4u + (uint32_t)i * 1024u;
        if (k < K) split_store4(xv[i], wv[i], scale, hr + k, lr + k);
    }
    for (uint32_t k = threadIdx.x * 4u + V * 1024u; k < K; k += 1024u)
        split_store4(*reinterpret_cast<const float4*>(xr + k), norm_w4(w, w_f32, k), scale, hr + k, lr + k);
}

// Adds the K splits and applies the epilogue. Thread (n, lane of 2) walks 8 activation rows of one problem.
// mode 0: C = sum (+ bias[n]) (+ residual[m][n]);  mode 1: problems 0/1 are gate/up, C = silu(gate) * up.
struct EpiArgs {
    const float* partial;
    float* out[3];
    const float* bias[3];
    const float* residual[3];
    uint32_t N[3];
    uint32_t tile_begin[4];
    uint32_t problems, M, n_total, k_splits, mode;
    uint32_t rope_on;
    M40TcRopeAppend rope;
};

__global__ void __launch_bounds__(256) gemm_tc_epilogue_kernel(EpiArgs e) {
    pdl_wait();
    pdl_trigger();
    const uint32_t p = blockIdx.z;
    const uint32_t n = blockIdx.x * 128u + (threadIdx.x & 127u);
    if (n >= e.N[p]) return;
    const size_t split_stride = (size_t)e.M * e.n_total;
    // a thread owns 4 activation rows; all partial loads of a chunk of splits are issued before any is used (the
    // additions keep the split order, so the result does not depend on timing)
    const uint32_t m0 = blockIdx.y * 8u + (threadIdx.x >> 7);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const size_t col = (size_t)e.tile_begin[p] * BLOCK_N + n;
    const size_t col_u = (size_t)e.tile_begin[1] * BLOCK_N + n;
    // Every load is unconditional (row and split index clamped, the value masked afterwards): guarded loads were
    // issued one at a time, each waiting for the previous one's trip to L2.
    const uint32_t M = e.M, ks = e.k_splits;
    const size_t n_total = e.n_total;
    const float* __restrict__ part = e.partial;
    const bool gate_up = e.mode == 1;
    for (uint32_t sbase = 0; sbase < ks; sbase += 4u) {
        float v[4][4], w[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t m = min(m0 + 2u * i, M - 1u), sp = min(sbase + k, ks - 1u);
                const size_t at = sp * split_stride + (size_t)m * n_total;
                v[i][k] = part[at + col];
                w[i][k] = gate_up ? part[at + col_u] : 0.0f;
            }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const bool live = sbase + k < ks;
                acc[i] += live ? v[i][k] : 0.0f;
                up[i] += live ? w[i][k] : 0.0f;
            }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t m = m0 + 2u * i;
        if (m >= e.M) continue;
        float r = acc[i];
        if (e.mode == 1) {
            e.out[0][(size_t)m * e.N[0] + n] = (r / (1.0f + expf(-r))) * up[i];
            continue;
        }
        if (e.bias[p]) r += e.bias[p][n];
        if (e.residual[p]) r += e.residual[p][(size_t)m * e.N[p] + n];
        if (!e.rope_on) {
            e.out[p][(size_t)m * e.N[p] + n] = r;
            continue;
        }
        // q | k | v tail (the whole warp is here: N is a multiple of 128 and m is the same for all lanes):
        // RoPE on adjacent pairs of q and k, then q to its buffer and k, v as f16 into the cache row of this position
        const M40TcRopeAppend& ra = e.rope;
        const uint32_t seq = ra.seq_ids[m], pos = ra.positions[m];
        const uint32_t d = n % ra.head_dim, head = n / ra.head_dim;
        const float other = __shfl_xor_sync(0xffffffffu, r, 1);
        if (seq >= ra.max_batch || pos >= ra.max_seq_len) {
            if (p == 0 && n == 0) atomicOr(ra.status, 2u);
            continue;
        }
        if (p < 2) {
            float c, sn;
            rope_cs(pos, d >> 1, ra.head_dim, ra.freq_base, ra.freq_scale, &c, &sn, ra.inv_freq);
            r = (d & 1u) ? other * sn + r * c : r * c - other * sn;
        }
        if (p == 0) {
            e.out[0][(size_t)m * e.N[0] + n] = r;
        } else {
            const size_t at = kv_row_offset(seq, head, pos, ra.kv_heads, ra.max_seq_len, ra.head_dim) + d;
            (p == 1 ? ra.d_k : ra.d_v)[at] = __float2half_rn(r);
            if (p == 1 && n == 0) ra.d_seq_map[seq] = pos + 1u;
        }
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

// 2D f16 tensor [rows][cols] row-major, box [box_rows][64], 128-byte swizzle, zero fill out of bounds.
bool make_map_f16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
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

}  // namespace

int m40_split_activations(M40llmCudaContext* ctx, cudaStream_t s, const float* X, __half* hi, __half* lo, int M, int K,
                          const M40GemvNorm* norm) {
    if (norm && norm->w) {
        if (K % 4 != 0 || (((uintptr_t)X) & 15u) != 0u) return -2;
        const bool w_vec = (((uintptr_t)norm->w) & (norm->w_is_f32 ? 15u : 7u)) == 0u;
        m40_launch_dependent(norm_split_rows_kernel, dim3((unsigned)M), dim3(256), 0, s, X, norm->w,
                             (norm->w_is_f32 ? 1 : 0) | (w_vec ? 0 : 2), norm->eps, hi, lo, (uint32_t)K);
    } else {
        const size_t n = (size_t)M * K;
        size_t blocks = (n + 255) / 256;
        if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
        m40_launch_dependent(split_activations_kernel, dim3((unsigned)blocks), dim3(256), 0, s, X, hi, lo, n);
    }
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

bool m40_gemm_tc_supported(int M, int K, int problems, const void* const* W) {
    if (M < 2 || M > 256 || K % 8 != 0 || K < BLOCK_K || problems < 1 || problems > 3) return false;
    for (int p = 0; p < problems; ++p)
        if ((((uintptr_t)W[p]) & 15u) != 0u) return false;
    return get_encode() != nullptr;
}

int m40_gemm_tc_f16(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* X, int M, int K,
                    int problems, const __half* const* W, const int* N, float* const* out, const float* const* bias,
                    const float* const* residual, int mode, const M40GemvNorm* norm, const M40TcRopeAppend* rope) {
    if (rope) {
        if (problems != 3 || mode != 0 || rope->head_dim == 0 || rope->head_dim % 2 != 0) return -2;
        for (int p = 0; p < 3; ++p)
            if (N[p] % 128 != 0 || N[p] % (int)rope->head_dim != 0) return -2;
    }
    const uint32_t M_pad = (uint32_t)((M + 15) / 16 * 16);
    TcArgs a = {};
    a.M = (uint32_t)M;
    a.M_pad = M_pad;
    a.K = (uint32_t)K;
    a.problems = (uint32_t)problems;
    // hi-only f16 activations miss the parity tolerance for outputs near zero (error ~3e-4 * |x| * sqrt(K) * |w|),
    // so the lo part is always carried; above ~128 rows this makes the kernel tensor-bound instead of HBM-bound.
    a.use_lo = 1u;
    uint32_t tiles = 0;
    for (int p = 0; p < problems; ++p) {
        a.tile_begin[p] = tiles;
        tiles += (uint32_t)((N[p] + BLOCK_N - 1) / BLOCK_N);
    }
    for (int p = problems; p < 4; ++p) a.tile_begin[p] = tiles;
    a.n_total = tiles * BLOCK_N;
    a.kblocks_total = (uint32_t)((K + BLOCK_K - 1) / BLOCK_K);
    // stages from the shared-memory budget; two CTAs per SM when the stage is small
    const uint32_t stage_bytes = BLOCK_N * BLOCK_K * 2 + (a.use_lo ? 2u : 1u) * M_pad * BLOCK_K * 2;
    uint32_t stages = (100u * 1024u) / stage_bytes;
    if (stages > 8) stages = 8;
    if (stages < 2) stages = 2;
    a.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + (2 * stages + 1) * 8 + 16 + 1024;
    const uint32_t ctas_per_sm = smem <= 110u * 1024u ? 2u : 1u;
    // K splits: fill about one wave of resident CTAs, keep at least 4 k-blocks per split
    uint32_t ks = ((uint32_t)ctx->sm_count * ctas_per_sm) / tiles;
    if (ks < 1) ks = 1;
    const uint32_t ks_max = a.kblocks_total / 4 ? a.kblocks_total / 4 : 1;
    if (ks > ks_max) ks = ks_max;
    if (ks > 16) ks = 16;
    a.kblocks_per_split = (a.kblocks_total + ks - 1) / ks;
    ks = (a.kblocks_total + a.kblocks_per_split - 1) / a.kblocks_per_split;

    // scratch: [hi][lo] activation copies, then the partials
    const size_t act_elems = (size_t)M * K;
    const size_t act_bytes = ((act_elems * 2 + 255) / 256) * 256;
    const size_t part_bytes = (size_t)ks * M * a.n_total * sizeof(float);
    unsigned char* scratch = (unsigned char*)m40_ensure_scratch(ctx, stream_kind, 2 * act_bytes + part_bytes);
    if (!scratch) return -2;
    __half* xh = (__half*)scratch;
    __half* xl = a.use_lo ? (__half*)(scratch + act_bytes) : nullptr;
    a.partial = (float*)(scratch + 2 * act_bytes);
    a.status = ctx->d_status;

    CUtensorMap mW[3], mXh, mXl;
    for (int p = 0; p < 3; ++p) {
        const int q = p < problems ? p : 0;
        if (!make_map_f16(&mW[p], W[q], (uint64_t)N[q], (uint64_t)K, BLOCK_N)) return -2;
    }
    if (!make_map_f16(&mXh, xh, (uint64_t)M, (uint64_t)K, M_pad)) return -2;
    if (!make_map_f16(&mXl, a.use_lo ? xl : xh, (uint64_t)M, (uint64_t)K, M_pad)) return -2;

    if (m40_split_activations(ctx, s, X, xh, xl, M, K, norm) != 0) return -2;
    static unsigned long long configured = 0ull;
    const unsigned long long bit = 1ull << (ctx->device_id & 63);
    if (!(configured & bit)) {
        if (cudaFuncSetAttribute(gemm_tc_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return -2;
        configured |= bit;
    }
    dim3 grid(tiles, ks);
    m40_launch_dependent(gemm_tc_f16_kernel, grid, dim3(192), smem, s, mW[0], mW[1], mW[2], mXh, mXl, a);
    M40_COUNT_LAUNCH(ctx);
    if (cudaGetLastError() != cudaSuccess) return -2;

    EpiArgs e = {};
    e.partial = a.partial;
    uint32_t maxN = 0;
    for (int p = 0; p < problems; ++p) {
        e.out[p] = out[p];
        e.bias[p] = bias ? bias[p] : nullptr;
        e.residual[p] = residual ? residual[p] : nullptr;
        e.N[p] = (uint32_t)N[p];
        if ((uint32_t)N[p] > maxN) maxN = (uint32_t)N[p];
    }
    for (int p = 0; p < 4; ++p) e.tile_begin[p] = a.tile_begin[p];
    e.problems = (uint32_t)problems;
    e.M = (uint32_t)M;
    e.n_total = a.n_total;
    e.k_splits = ks;
    e.mode = (uint32_t)mode;
    if (rope) {
        e.rope_on = 1u;
        e.rope = *rope;
    }
    dim3 egrid((maxN + 127) / 128, (unsigned)(M + 7) / 8, mode == 1 ? 1u : (unsigned)problems);
    m40_launch_dependent(gemm_tc_epilogue_kernel, egrid, dim3(256), 0, s, e);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
