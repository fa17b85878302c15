// Single-row GEMV over streamed weights (decode batch 1): out[n] = x . W[n].
//
// At one activation row every weight byte is read once and nothing is reused, so the only thing that matters is
// keeping HBM busy. The kernel is persistent (one CTA per SM) and warp-specialised:
//
//   * two producer threads (one per producer warp, alternating stages: arming a stage costs one thread more than a
//     stage's share of the HBM time) stream groups of whole weight rows into a shared-memory ring with 1-D bulk async
//     copies (cp.async.bulk ... mbarrier::complete_tx), 8-36 KB per stage and up to ~200 KB in flight per SM,
//     independent of how fast the consumers issue instructions. Every CTA gets the same number of stages: the
//     group count is made a multiple of the grid by cutting the tail of the last matrix into groups one row smaller;
//   * sixteen consumer warps form groups of `cw` warps; a group owns every G-th stage, so the groups run
//     decoupled from one another (no CTA-wide barrier in the steady state). A thread owns fixed column pieces of
//     every row, so its slice of the activation vector stays in registers for the whole launch:
//       - f16 weights: 16-byte pieces, f32 activations, f32 FMAs;
//       - Q8_0 weights: 68-byte pieces (two raw 34-byte GGUF blocks: 4-byte aligned although single blocks are
//         not), int8 dot products with dp4a against the activations held as three signed 8-bit digits per value
//         and one scale per 32-block (x = s/128 * (128 a + b + c/128), error <= 2^-22 of the block maximum, i.e.
//         f32 rounding level), then one f32 multiply-add per block with d * s. The digits are made once per CTA
//         (cooperatively, into shared memory) with add-magic rounding, so no conversion-unit instruction is used;
//         once every consumer holds its slice in registers that shared memory is handed to the ring's last slots;
//   * row sums meet by warp shuffle, then across the warps of the group through shared memory in a fixed
//     order (no atomics: results are deterministic).
// Up to three matrices that share x go in one launch (Wq | Wk | Wv), gate and up are streamed side by side with
// the SwiGLU epilogue, bias/residual are folded into the store, and the RMSNorm of x can be applied on the fly.
//
// Every wait is bounded: a wait that runs out raises bit 4 of the context's status word, the CTA stops consuming
// (all warps still pass the same barriers) and drains its own copies before it returns.
#include "gemv_stream.cuh"

#include <stdlib.h>

#include "tc_ptx.cuh"

namespace {
using namespace tc;

constexpr int CWARPS = 16;                // consumer warps
constexpr int CONSUMERS = CWARPS * 32;
constexpr int PWARPS = 2;                 // producer warps (one elected thread each)
constexpr int THREADS = CONSUMERS + 32 * PWARPS;
constexpr int MAX_SEGS = 4;  // three matrices + the tail part of the last one
constexpr int MAX_STAGES = 12;
constexpr int MAX_ROWS = 16;              // rows of one matrix per stage
constexpr uint32_t STAGE_MAX = 36u * 1024u;
constexpr uint32_t SMEM_MAX = 200u * 1024u;  // ring + activation digits

struct SegDev {
    const uint8_t* W;
    const uint8_t* W2;
    float* out;
    const float* bias;
    const float* residual;
    int N;
    int group0;  // id of this matrix's first row group
    int R;       // rows per group of this matrix (the last group may hold fewer)
};

struct GemvArgs {
    SegDev seg[MAX_SEGS];
    const float* x;
    const void* norm_w;
    float* xn_out;
    uint32_t* status;
    float eps;
    int norm_f32;
    int nseg, K, pieces, cw, R, nstages, total_groups;
    uint32_t row_bytes, stage_bytes, xq_off;
    int first_late;  // ring slots from this one on share their bytes with the activation digits
};

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }
// Barrier of one consumer group (ids 2..9; id 1 is the all-consumer barrier, id 0 __syncthreads).
__device__ __forceinline__ void group_barrier(int grp, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(grp + 2), "r"(threads) : "memory");
}

__device__ __forceinline__ void locate_group(const GemvArgs& a, int g, int* seg, int* row0, int* rows) {
    int s = 0;
#pragma unroll
    for (int i = 1; i < MAX_SEGS; ++i)
        if (i < a.nseg && g >= a.seg[i].group0) s = i;
    const int r0 = (g - a.seg[s].group0) * a.seg[s].R;
    const int left = a.seg[s].N - r0;
    *seg = s;
    *row0 = r0;
    *rows = left < a.seg[s].R ? left : a.seg[s].R;
}

__device__ __forceinline__ float dot8(const uint4& w, const float* x) {
    const __half2* h = reinterpret_cast<const __half2*>(&w);
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        acc = fmaf(x[2 * i], f.x, acc);
        acc = fmaf(x[2 * i + 1], f.y, acc);
    }
    return acc;
}

// Activations of one 64-value piece as three int8 digits per value (packed 4 per word) and a scale per 32-block.
struct Q80X {
    int d[3][16];
    float s[2];
};

// Four values -> one word of each of the three digit planes. v * (127 * 2^14 / block maximum) + 1.5 * 2^23 leaves the
// rounded 22-bit integer q (ties to even, like rintf) in the low mantissa bits as two's complement; its base-128
// digits are q = 16384 a + 128 b + c with a = q >> 14 in [-127, 127] (floor) and b, c in [0, 127]: shifts and byte
// picks, no conversion instruction.
__device__ __forceinline__ void q80_quantise_unit(const float4& v, float inv14, uint32_t* pa, uint32_t* pb, uint32_t* pc) {
    const float MAGIC = 12582912.0f;
    const uint32_t m0 = __float_as_uint(fmaf(v.x, inv14, MAGIC)), m1 = __float_as_uint(fmaf(v.y, inv14, MAGIC));
    const uint32_t m2 = __float_as_uint(fmaf(v.z, inv14, MAGIC)), m3 = __float_as_uint(fmaf(v.w, inv14, MAGIC));
    // low byte of each of the four words -> one packed word
    auto pack = [](uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
        return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
    };
    *pc = pack(m0, m1, m2, m3) & 0x7f7f7f7fu;
    *pb = pack(m0 >> 7, m1 >> 7, m2 >> 7, m3 >> 7) & 0x7f7f7f7fu;
    *pa = pack(m0 >> 14, m1 >> 14, m2 >> 14, m3 >> 14);
}

// RMSNorm weights k .. k+3 as f32 (f32 or f16 storage, 16- resp. 8-byte aligned: k is a multiple of 4).
__device__ __forceinline__ float4 load_norm4(const void* w, int is_f32, int k) {
    if (is_f32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + k);
    const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(w) + k);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// x . (two raw Q8_0 blocks at a 4-byte aligned shared-memory address).
__device__ __forceinline__ float q80_pair_dot(const uint32_t* wp, const Q80X& x) {
    uint32_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = wp[i];
    int sa = 0, sb = 0, sc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // first block: scale in the low half of w[0], weights from byte 2
        const int q = (int)__funnelshift_r(w[i], w[i + 1], 16);
        sa = __dp4a(q, x.d[0][i], sa);
        sb = __dp4a(q, x.d[1][i], sb);
        sc = __dp4a(q, x.d[2][i], sc);
    }
    const float d0 = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xffffu)));
    float r = fmaf((float)sc, 1.0f / 128.0f, (float)(sa * 128 + sb)) * (d0 * x.s[0]);
    sa = sb = sc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // second block: scale in the high half of w[8], weights word aligned
        const int q = (int)w[9 + i];
        sa = __dp4a(q, x.d[0][8 + i], sa);
        sb = __dp4a(q, x.d[1][8 + i], sb);
        sc = __dp4a(q, x.d[2][8 + i], sc);
    }
    const float d1 = __half2float(__ushort_as_half((unsigned short)(w[8] >> 16)));
    return fmaf(fmaf((float)sc, 1.0f / 128.0f, (float)(sa * 128 + sb)), d1 * x.s[1], r);
}

// bias[n] + residual[n]: loaded at the top of a stage so that the latency hides behind the dot products.
__device__ __forceinline__ float load_addend(const SegDev& sg, int n) {
    float add = 0.0f;
    if (sg.bias) add = sg.bias[n];
    if (sg.residual) add += sg.residual[n];
    return add;
}

template <int GATE_UP>
__device__ __forceinline__ void store_row(const SegDev& sg, int n, float v, float v2, float add) {
    if (GATE_UP) v = (v / (1.0f + expf(-v))) * v2;
    sg.out[n] = v + add;
}

template <int FMT, int GATE_UP, int CPT>
__global__ void __launch_bounds__(THREADS, 1) gemv_stream_kernel(const __grid_constant__ GemvArgs a) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full[MAX_STAGES], empty[MAX_STAGES], xq_done;
    __shared__ float red[2][2][MAX_ROWS][CWARPS];  // [parity][matrix][row][consumer warp]
    __shared__ float ssq[CWARPS];
    __shared__ volatile uint32_t abort_flag;
    // use number (ring index / nstages) the producer last armed each slot for: a parity wait can only tell adjacent
    // uses of a slot apart, and a group may reach a slot that another group used last
    __shared__ volatile uint32_t slot_use[MAX_STAGES];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < a.nstages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
            slot_use[s] = 0xffffffffu;
        }
        mbar_init(&xq_done, CWARPS);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();  // the successor may be placed as soon as this CTA's resources free up
    const int my_groups = ((int)blockIdx.x < a.total_groups)
                              ? (a.total_groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const uint32_t mat2_off = (uint32_t)a.R * a.row_bytes;

    if (warp >= CWARPS) {
        // ------------------------------------------------------------ producers
        // Arming a stage (barrier transaction count + the bulk copies) costs one thread several hundred cycles, more
        // than a stage's share of the HBM time, so the stages are dealt to PWARPS threads.
        if (lane != 0) return;
        const int pw = warp - CWARPS;
        int issued = pw;  // first stage of this thread not yet issued
        int s = pw;       // ring slot and use number of stage i, carried (no division in this loop)
        uint32_t use = 0;
        for (int i = pw; i < my_groups; i += PWARPS) {
            bool ready = true;
            if (use > 0) {
                // the slot's previous use may have been armed by the other producer thread: only once that has
                // happened does the parity of the release barrier mean the release of THAT use
                for (uint32_t spin = 0; slot_use[s] != use - 1u && spin < WAIT_LIMIT; ++spin) {}
                ready = slot_use[s] == use - 1u && mbar_wait(&empty[s], (use & 1u) ^ 1u);
            } else if (s >= a.first_late) {
                ready = mbar_wait(&xq_done, 0u);  // the consumers have taken their digits out of these bytes
            }
            if (!ready) {
                abort_flag = 1;
                atomicOr(a.status, 4u);
                break;
            }
            if (abort_flag) break;
            int sidx, row0, rows;
            locate_group(a, (int)blockIdx.x + i * (int)gridDim.x, &sidx, &row0, &rows);
            const SegDev& sg = a.seg[sidx];
            const uint32_t bytes = (uint32_t)rows * a.row_bytes;
            uint8_t* dst = ring + (size_t)s * a.stage_bytes;
            // No fence between the two: once the consumers have released the previous use (waited for above) the
            // barrier is in this use's phase, so a consumer that sees the new use number early merely waits.
            slot_use[s] = use;
            mbar_expect_tx(&full[s], GATE_UP ? 2u * bytes : bytes);
            bulk_load(dst, sg.W + (size_t)row0 * a.row_bytes, bytes, &full[s]);
            if (GATE_UP) bulk_load(dst + mat2_off, sg.W2 + (size_t)row0 * a.row_bytes, bytes, &full[s]);
            issued = i + PWARPS;
            s += PWARPS;
            if (s >= a.nstages) s -= a.nstages, ++use;
        }
        if (abort_flag) {
            // the consumers have stopped: wait (bounded) for this thread's copies still in flight before the CTA
            // goes away
            int first = issued - a.nstages;
            if (first < pw) first = pw;
            for (int i = first; i < issued; i += PWARPS) mbar_wait(&full[i % a.nstages], (uint32_t)((i / a.nstages) & 1));
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    // The weights streamed by the producer above never depend on the previous kernel; the activations do.
    pdl_wait();
    const int cw = a.cw, G = CWARPS / cw;
    const int grp = warp / cw, cwi = warp % cw;
    const int c = cwi * 32 + lane, cols = cw * 32;

    float xr[FMT == M40_GEMV_Q80 ? 1 : CPT][8];
    Q80X xq;
    float scale = 1.0f;
    if (FMT == M40_GEMV_Q80) {
        // Digits of the whole row, once per CTA. A thread takes 4-value units tid, tid + 512, ...: coalesced 16-byte
        // loads, one word per digit plane per unit, and the eight units of a 32-block sit in eight adjacent lanes.
        // Shared layout: [plane][word quad i4][piece][4 words], rows padded by 8 words, so that both these stores
        // and the 16-byte reads of a thread's own piece below are free of bank conflicts.
        uint32_t* dig = reinterpret_cast<uint32_t*>(ring + a.xq_off);
        const int prow = a.pieces * 4 + 8;
        float* xs = reinterpret_cast<float*>(dig + 12 * prow);  // [K/32]
        const int units = a.K / 4;
        constexpr int UR = 8;  // units per thread and round; with a norm the host admits one round only
        for (int u0 = 0; u0 < units; u0 += CONSUMERS * UR) {
            float4 xv[UR], wv[UR];
#pragma unroll
            for (int p = 0; p < UR; ++p) {
                const int u = u0 + p * CONSUMERS + tid;
                xv[p] = u < units ? *reinterpret_cast<const float4*>(a.x + 4 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
                if (a.norm_w) wv[p] = u < units ? load_norm4(a.norm_w, a.norm_f32, 4 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (a.norm_w) {
                float ss = 0.0f;
#pragma unroll
                for (int p = 0; p < UR; ++p)
                    ss += xv[p].x * xv[p].x + xv[p].y * xv[p].y + xv[p].z * xv[p].z + xv[p].w * xv[p].w;
                ss = warp_sum(ss);
                if (lane == 0) ssq[warp] = ss;
                consumer_barrier();
                float tot = 0.0f;
#pragma unroll
                for (int i = 0; i < CWARPS; ++i) tot += ssq[i];
                scale = rsqrtf(tot / (float)a.K + a.eps);
            }
#pragma unroll
            for (int p = 0; p < UR; ++p) {
                const int u = u0 + p * CONSUMERS + tid;
                if (u0 + p * CONSUMERS + warp * 32 >= units) break;  // whole warps: units is a multiple of 64
                float4 v = xv[p];
                if (a.norm_w) {
                    v.x = v.x * scale * wv[p].x, v.y = v.y * scale * wv[p].y;
                    v.z = v.z * scale * wv[p].z, v.w = v.w * scale * wv[p].w;
                    if (a.xn_out && blockIdx.x == 0 && u < units) *reinterpret_cast<float4*>(a.xn_out + 4 * u) = v;
                }
                float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                const float inv14 = mx > 0.0f ? (127.0f * 16384.0f) / mx : 0.0f;
                uint32_t da, db, dc;
                q80_quantise_unit(v, inv14, &da, &db, &dc);
                if (u < units) {
                    const int pc = u >> 4, j = u & 15;
                    uint32_t* dst = dig + (j >> 2) * prow + pc * 4 + (j & 3);
                    dst[0] = da, dst[4 * prow] = db, dst[8 * prow] = dc;
                    if ((u & 7) == 0) xs[u >> 3] = mx * (1.0f / (127.0f * 128.0f));
                }
            }
        }
        consumer_barrier();
#pragma unroll
        for (int i = 0; i < 16; ++i) xq.d[0][i] = xq.d[1][i] = xq.d[2][i] = 0;
        xq.s[0] = xq.s[1] = 0.0f;
        if (c < a.pieces) {
#pragma unroll
            for (int pl = 0; pl < 3; ++pl)
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const uint4 t = *reinterpret_cast<const uint4*>(dig + (pl * 4 + (i >> 2)) * prow + c * 4);
                    xq.d[pl][i] = (int)t.x, xq.d[pl][i + 1] = (int)t.y, xq.d[pl][i + 2] = (int)t.z, xq.d[pl][i + 3] = (int)t.w;
                }
            const float2 sc2 = *reinterpret_cast<const float2*>(xs + 2 * c);
            xq.s[0] = sc2.x, xq.s[1] = sc2.y;
        }
        // The digit area is dead from here on: the last ring slots lie over it. Order this thread's reads before the
        // bulk copies (async proxy) that will overwrite them, then tell the producers.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&xq_done);
    } else {
        float4 sv[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
        float4 wr[CPT][2];
        if (a.norm_w) {  // the loads of the sum-of-squares pass and of this thread's own pieces go out together
            const int k = tid * 4;
            if (k < a.K) sv[0] = *reinterpret_cast<const float4*>(a.x + k);
            if (k + CONSUMERS * 4 < a.K) sv[1] = *reinterpret_cast<const float4*>(a.x + k + CONSUMERS * 4);
        }
#pragma unroll
        for (int j = 0; j < CPT; ++j) {
            const int p = c + j * cols;
#pragma unroll
            for (int i = 0; i < 8; ++i) xr[j][i] = 0.0f;
            wr[j][0] = wr[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p < a.pieces) {
                const int k0 = p * 8;
                const float4 t0 = *reinterpret_cast<const float4*>(a.x + k0);
                const float4 t1 = *reinterpret_cast<const float4*>(a.x + k0 + 4);
                xr[j][0] = t0.x, xr[j][1] = t0.y, xr[j][2] = t0.z, xr[j][3] = t0.w;
                xr[j][4] = t1.x, xr[j][5] = t1.y, xr[j][6] = t1.z, xr[j][7] = t1.w;
                if (a.norm_w) {
                    wr[j][0] = load_norm4(a.norm_w, a.norm_f32, k0);
                    wr[j][1] = load_norm4(a.norm_w, a.norm_f32, k0 + 4);
                }
            }
        }
        if (a.norm_w) {
            float ss = sv[0].x * sv[0].x + sv[0].y * sv[0].y + sv[0].z * sv[0].z + sv[0].w * sv[0].w +
                       sv[1].x * sv[1].x + sv[1].y * sv[1].y + sv[1].z * sv[1].z + sv[1].w * sv[1].w;
            for (int k = tid * 4 + 2 * CONSUMERS * 4; k < a.K; k += CONSUMERS * 4) {
                const float4 v = *reinterpret_cast<const float4*>(a.x + k);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss = warp_sum(ss);
            if (lane == 0) ssq[warp] = ss;
            consumer_barrier();
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < CWARPS; ++i) tot += ssq[i];
            scale = rsqrtf(tot / (float)a.K + a.eps);
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                const int p = c + j * cols;
                const float w8[8] = {wr[j][0].x, wr[j][0].y, wr[j][0].z, wr[j][0].w,
                                     wr[j][1].x, wr[j][1].y, wr[j][1].z, wr[j][1].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) xr[j][i] = xr[j][i] * scale * w8[i];
                if (p < a.pieces && a.xn_out && blockIdx.x == 0 && grp == 0) {
                    const int k0 = p * 8;
                    *reinterpret_cast<float4*>(a.xn_out + k0) = make_float4(xr[j][0], xr[j][1], xr[j][2], xr[j][3]);
                    *reinterpret_cast<float4*>(a.xn_out + k0 + 4) = make_float4(xr[j][4], xr[j][5], xr[j][6], xr[j][7]);
                }
            }
        }
    }

    constexpr uint32_t PIECE_BYTES = FMT == M40_GEMV_Q80 ? 68u : 16u;
    int it = 0;  // this group's stage counter (parity of the reduction buffer)
    int s = grp % a.nstages;  // ring slot and use number of stage i, carried from stage to stage
    uint32_t use = (uint32_t)(grp / a.nstages);
    for (int i = grp; i < my_groups; i += G, ++it) {
        if (i != grp) {
            s += G;
            while (s >= a.nstages) s -= a.nstages, ++use;
        }
        bool ok = abort_flag == 0;
        if (ok) {  // the slot must be armed for THIS use before its parity means anything
            for (uint32_t spin = 0; slot_use[s] != use && spin < WAIT_LIMIT; ++spin) {}
            ok = slot_use[s] == use;
        }
        if (!ok || !mbar_wait(&full[s], use & 1u)) {
            abort_flag = 1;
            if (lane == 0) atomicOr(a.status, 4u);
            ok = false;
        }
        int sidx, row0, rows;
        locate_group(a, (int)blockIdx.x + i * (int)gridDim.x, &sidx, &row0, &rows);
        const SegDev& sg = a.seg[sidx];
        const uint8_t* st = ring + (size_t)s * a.stage_bytes;
        float add_final = 0.0f;
        if (cw > 1 && ok && c < rows) add_final = load_addend(sg, row0 + c);
        if (ok) {
            for (int r = 0; r < rows; r += 2) {  // two rows per pass: independent chains for the shuffles
                const bool two = r + 1 < rows;
                const uint8_t* rowp = st + (size_t)r * a.row_bytes;
                float acc[2] = {0.0f, 0.0f}, acc2[2] = {0.0f, 0.0f}, add[2] = {0.0f, 0.0f};
                if (cw == 1 && lane == 0) {
                    add[0] = load_addend(sg, row0 + r);
                    if (two) add[1] = load_addend(sg, row0 + r + 1);
                }
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    const int p = c + j * cols;
                    if (p < a.pieces) {
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            if (rr == 1 && !two) break;
                            const uint8_t* pp = rowp + (size_t)rr * a.row_bytes + (size_t)p * PIECE_BYTES;
                            if (FMT == M40_GEMV_Q80) {
                                acc[rr] += q80_pair_dot(reinterpret_cast<const uint32_t*>(pp), xq);
                                if (GATE_UP) acc2[rr] += q80_pair_dot(reinterpret_cast<const uint32_t*>(pp + mat2_off), xq);
                            } else {
                                acc[rr] += dot8(*reinterpret_cast<const uint4*>(pp), xr[j]);
                                if (GATE_UP) acc2[rr] += dot8(*reinterpret_cast<const uint4*>(pp + mat2_off), xr[j]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    acc[rr] = warp_sum(acc[rr]);
                    if (GATE_UP) acc2[rr] = warp_sum(acc2[rr]);
                }
                if (lane == 0) {
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        if (rr == 1 && !two) break;
                        if (cw == 1) {
                            store_row<GATE_UP>(sg, row0 + r + rr, acc[rr], acc2[rr], add[rr]);
                        } else {
                            red[it & 1][0][r + rr][warp] = acc[rr];
                            if (GATE_UP) red[it & 1][1][r + rr][warp] = acc2[rr];
                        }
                    }
                }
            }
        }
        if (cw > 1) {
            group_barrier(grp, cols);  // every warp of the group has read the stage and written its partials
            if (c == 0) mbar_arrive(&empty[s]);
            if (ok && c < rows) {
                float v = 0.0f, v2 = 0.0f;
                for (int k = 0; k < cw; ++k) {
                    v += red[it & 1][0][c][grp * cw + k];
                    if (GATE_UP) v2 += red[it & 1][1][c][grp * cw + k];
                }
                store_row<GATE_UP>(sg, row0 + c, v, v2, add_final);
            }
        } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
    }
}

template <int FMT, int GATE_UP, int CPT>
int launch(M40llmCudaContext* ctx, cudaStream_t s, const GemvArgs& a, int grid, size_t smem) {
    static bool attr_set[64] = {};
    const int dev = ctx->device_id;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(gemv_stream_kernel<FMT, GATE_UP, CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM_MAX) != cudaSuccess)
            return -2;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const cudaError_t e = m40_launch_dependent(gemv_stream_kernel<FMT, GATE_UP, CPT>, dim3(grid), dim3(THREADS), smem, s, a);
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -2;
}

template <int GATE_UP>
int launch_fmt(M40llmCudaContext* ctx, cudaStream_t s, const GemvArgs& a, int grid, size_t smem, int fmt, int cpt) {
    if (fmt == M40_GEMV_Q80) return launch<M40_GEMV_Q80, GATE_UP, 1>(ctx, s, a, grid, smem);
    if (cpt == 1) return launch<M40_GEMV_F16, GATE_UP, 1>(ctx, s, a, grid, smem);
    if (cpt == 2) return launch<M40_GEMV_F16, GATE_UP, 2>(ctx, s, a, grid, smem);
    if (cpt == 4) return launch<M40_GEMV_F16, GATE_UP, 4>(ctx, s, a, grid, smem);
    return 1;
}

bool aligned16(const void* p) { return (((uintptr_t)p) & 15u) == 0u; }

}  // namespace

int m40_gemv_stream(M40llmCudaContext* ctx, cudaStream_t s, const float* x, int K, int fmt, int gate_up, int nseg,
                    const M40GemvSeg* segs, const M40GemvNorm* norm) {
    if (nseg < 1 || nseg > MAX_SEGS - 1 || K <= 0 || !aligned16(x)) return 1;
    GemvArgs a = {};
    int cpt_max;
    uint32_t xq_bytes = 0;
    if (fmt == M40_GEMV_F16) {
        if (K % 8 != 0) return 1;
        a.row_bytes = (uint32_t)K * 2u;
        a.pieces = K / 8;
        cpt_max = 4;
    } else if (fmt == M40_GEMV_Q80) {
        if (K % 256 != 0) return 1;  // whole block pairs and 16-byte row pitch
        a.row_bytes = (uint32_t)(K / 32) * 34u;
        a.pieces = K / 64;
        cpt_max = 1;
        xq_bytes = (uint32_t)(12 * (K / 16 + 8) * 4 + (K / 32) * 4);  // 3 planes x 4 padded rows + block scales
        if (norm && norm->w && K > CONSUMERS * 8 * 4) return 1;      // the norm needs the whole row in one register round
        xq_bytes = (xq_bytes + 127u) & ~127u;
    } else {
        return 1;
    }
    const uint32_t nmat = gate_up ? 2u : 1u;
    for (int i = 0; i < nseg; ++i) {
        if (segs[i].N <= 0 || !segs[i].W || !segs[i].out || !aligned16(segs[i].W)) return 1;
        if (gate_up && (!segs[i].W2 || !aligned16(segs[i].W2))) return 1;
    }
    if (norm && norm->w && (!aligned16(norm->w) || (norm->xn_out && !aligned16(norm->xn_out)))) return 1;
    if ((uint64_t)a.row_bytes * nmat > STAGE_MAX || xq_bytes + 2u * a.row_bytes * nmat > SMEM_MAX) return 1;
    // the digits are only needed until every consumer holds its slice in registers: the last ring slots reuse their bytes

    // Warps per group: the fewest whose per-thread register slice of x fits.
    int cw = 0, cpt = 0;
    for (int w = 1; w <= CWARPS; w *= 2) {
        const int need = (a.pieces + w * 32 - 1) / (w * 32);
        int p2 = 1;
        while (p2 < need) p2 *= 2;
        if (p2 > cpt_max) continue;
        cw = w;
        cpt = p2;
        break;
    }
    if (!cw) return 1;
    const int G = CWARPS / cw;
    const uint32_t ring_max = SMEM_MAX;

    // Rows per stage: within the stage budget, a ring deep enough that every group can hold a stage while two
    // more are in flight (when the row size allows), and among those the choice that loads the persistent CTAs
    // most evenly (ties: the larger stage).
    const int grid_max = ctx->sm_count > 0 ? ctx->sm_count : 1;
    int best_R = 0;
    {
        double eff_of[MAX_ROWS + 1];
        int deep_of[MAX_ROWS + 1];
        int n_cand = 0, any_deep = 0;
        double best_eff = -1.0;
        for (int R = 1; R <= MAX_ROWS; ++R) {
            const uint64_t sb = ((uint64_t)R * a.row_bytes * nmat + 127u) & ~(uint64_t)127u;
            if (sb > STAGE_MAX) break;
            long long nst = (long long)(ring_max / sb);
            if (nst > MAX_STAGES) nst = MAX_STAGES;
            if (nst < 2) break;
            long long groups = 0;
            for (int i = 0; i < nseg; ++i) groups += (segs[i].N + R - 1) / R;
            const long long grid = groups < grid_max ? groups : grid_max;
            const long long per = (groups + grid - 1) / grid;
            eff_of[R] = (double)groups / (double)(per * grid);
            deep_of[R] = nst >= G + 2 ? 1 : 0;
            any_deep |= deep_of[R];
            n_cand = R;
        }
        for (int R = 1; R <= n_cand; ++R)
            if (deep_of[R] == any_deep && eff_of[R] > best_eff) best_eff = eff_of[R];
        // the largest stage within 3 % of the best balance: fewer barrier round trips per byte
        for (int R = 1; R <= n_cand; ++R)
            if (deep_of[R] == any_deep && eff_of[R] >= best_eff - 0.03) best_R = R;
    }
    if (!best_R) return 1;
    a.R = best_R;
    a.cw = cw;
    a.stage_bytes = ((uint32_t)a.R * a.row_bytes * nmat + 127u) & ~127u;
    a.nstages = (int)(ring_max / a.stage_bytes);
    if (a.nstages > MAX_STAGES) a.nstages = MAX_STAGES;
    if (a.nstages < 2) return 1;
    // shared memory: [ring slots ...], the digits right-aligned over the last slots (or behind a short ring)
    uint32_t smem_bytes = (uint32_t)a.nstages * a.stage_bytes;
    if (smem_bytes < xq_bytes + 2u * a.stage_bytes) smem_bytes = xq_bytes + 2u * a.stage_bytes;  // >= 2 early slots
    if (smem_bytes > SMEM_MAX) return 1;
    a.xq_off = smem_bytes - xq_bytes;
    a.first_late = xq_bytes ? (int)(a.xq_off / a.stage_bytes) : a.nstages;
    // Row groups: a.R rows each, dealt round-robin to the CTAs. So that every CTA gets the same number of stages (a
    // CTA with one stage more than the rest finishes a memory round trip late while the others idle), the group
    // count is raised to the next multiple of the CTA count by giving the tail of the last matrix groups of
    // a.R - 1 rows: x groups of R and y of R - 1 rows with x + y = groups and R x + (R - 1) y = N.
    int g = 0, nout = 0;
    long long groups_other = 0;
    for (int i = 0; i + 1 < nseg; ++i) groups_other += (segs[i].N + a.R - 1) / a.R;
    const int last_N = segs[nseg - 1].N;
    const long long groups0 = groups_other + (last_N + a.R - 1) / a.R;
    int tail_groups = 0;  // y
    if (groups0 > grid_max && groups0 % grid_max != 0 && a.R >= 2 && last_N % a.R == 0) {
        const long long want = (groups0 + grid_max - 1) / grid_max * grid_max - groups_other;
        const long long y = (long long)a.R * want - last_N;
        if (y > 0 && y <= want) tail_groups = (int)y;
    }
    const int tail_rows = tail_groups * (a.R - 1);
    for (int i = 0; i < nseg; ++i) {
        const int main_rows = i == nseg - 1 ? segs[i].N - tail_rows : segs[i].N;
        for (int part = 0; part < 2; ++part) {
            const int r0 = part == 0 ? 0 : main_rows;
            const int n = part == 0 ? main_rows : segs[i].N - main_rows;
            if (n <= 0) continue;
            SegDev& d = a.seg[nout++];
            d.W = (const uint8_t*)segs[i].W + (size_t)r0 * a.row_bytes;
            d.W2 = segs[i].W2 ? (const uint8_t*)segs[i].W2 + (size_t)r0 * a.row_bytes : nullptr;
            d.out = segs[i].out + r0;
            d.bias = segs[i].bias ? segs[i].bias + r0 : nullptr;
            d.residual = segs[i].residual ? segs[i].residual + r0 : nullptr;
            d.N = n;
            d.group0 = g;
            d.R = part == 0 ? a.R : a.R - 1;
            g += (n + d.R - 1) / d.R;
        }
    }
    nseg = nout;
    a.nseg = nseg;
    a.total_groups = g;
    a.K = K;
    a.x = x;
    a.status = ctx->d_status;
    if (norm && norm->w) {
        a.norm_w = norm->w;
        a.norm_f32 = norm->w_is_f32;
        a.eps = norm->eps;
        a.xn_out = norm->xn_out;
    }
    const int grid = g < grid_max ? g : grid_max;
    const size_t smem = smem_bytes;
    return gate_up ? launch_fmt<1>(ctx, s, a, grid, smem, fmt, cpt) : launch_fmt<0>(ctx, s, a, grid, smem, fmt, cpt);
}

