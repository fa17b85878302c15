/*
 * CPU oracle for the m40-llm per-token decode path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA library: it
 * restates, in plain C with f32 arithmetic and the reference's loop order, the
 * CPU math that the reference project uses to validate the same operations.
 * Nothing in the product library links, calls or falls back to this code.
 *
 * Pinning: every function below is checked (tests/test_oracle_*.py) against
 * golden outputs produced by the reference project's own CUDA translation unit
 * (cuda/kernels.cu compiled unmodified by `make -C oracle ref`) on a B200,
 * committed under tests/golden/, and against an independent numpy restatement
 * of the reference tests' closed-form cases.
 *
 * Each function cites the reference file:line it follows (paths are relative
 * to the reference project's root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- f16 <-> f32
 * IEEE binary16 round-to-nearest-even, the arithmetic of half::f16::from_f32
 * (crate `half` 2.7.1, Cargo.lock:599) used at src/cuda.rs:3625-3628 and of
 * __float2half_rn in cuda/kernels.cu:5550. */
ORC_API uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | (absx > 0x7f800000u ? 0x0200u | ((absx >> 13) & 0x3ffu) : 0u));
    }
    if (absx >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or == 2^-25 tie -> even = 0) */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u; /* 24-bit significand */
    uint32_t shift;
    uint32_t half_exp;
    if (exp < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(exp + 15);
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q += 1u;
    uint32_t out;
    if (half_exp == 0) {
        out = q; /* may carry into exponent 1: correct by construction */
    } else {
        out = ((half_exp - 1u) << 10) + q; /* q includes the implicit bit (0x400) */
    }
    return (uint16_t)(sign | out);
}

ORC_API float orc_f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    const uint32_t man = h & 0x3ffu;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            float v = (float)man * (1.0f / 16777216.0f); /* man * 2^-24 */
            memcpy(&x, &v, 4);
            x |= sign;
        }
    } else if (exp == 31) {
        x = sign | 0x7f800000u | (man << 13);
    } else {
        x = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

ORC_API void orc_f32_to_f16_array(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = orc_f32_to_f16(in[i]);
}

ORC_API void orc_f16_to_f32_array(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = orc_f16_to_f32(in[i]);
}

/* ------------------------------------------------------------------- RMSNorm
 * tests/rmsnorm_rope.rs:9-40 (sequential f32 sum of squares,
 * scale = 1/sqrt(sum/dim + eps), out = (x*scale)*w); device form
 * cuda/kernels.cu:770-807. `w` may be NULL (unweighted, kernels.cu:736-768). */
ORC_API void orc_rms_norm(const float* in, const float* w, float* out, size_t rows, size_t dim, float eps) {
    for (size_t r = 0; r < rows; ++r) {
        const float* x = in + r * dim;
        float ss = 0.0f;
        for (size_t i = 0; i < dim; ++i) ss += x[i] * x[i];
        const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
        for (size_t i = 0; i < dim; ++i) {
            float v = x[i] * scale;
            if (w) v *= w[i];
            out[r * dim + i] = v;
        }
    }
}

/* ---------------------------------------------------------------------- RoPE
 * Adjacent pairs: tests/rmsnorm_rope.rs:43-76. NeoX split-half pairing:
 * cuda/kernels.cu:5570-5585 (pair i of a head = elements (i, i+hd/2)).
 * theta = float(pos)*freq_scale * powf(base, -2 i / hd)  (kernels.cu:7322-7331).
 * layout 0 = adjacent, 1 = NeoX. Position of row r is past_len + r. */
ORC_API void orc_rope(float* x, size_t rows, size_t heads, size_t head_dim, uint32_t past_len,
                      float freq_base, float freq_scale, uint32_t layout) {
    const size_t half = head_dim / 2;
    for (size_t r = 0; r < rows; ++r) {
        const float pos = (float)(past_len + (uint32_t)r) * freq_scale;
        for (size_t h = 0; h < heads; ++h) {
            float* xh = x + (r * heads + h) * head_dim;
            for (size_t i = 0; i < half; ++i) {
                const float theta = pos * powf(freq_base, -2.0f * (float)i / (float)head_dim);
                const float c = cosf(theta);
                const float s = sinf(theta);
                const size_t i0 = layout == 1u ? i : 2 * i;
                const size_t i1 = layout == 1u ? i + half : 2 * i + 1;
                const float a = xh[i0];
                const float b = xh[i1];
                xh[i0] = a * c - b * s;
                xh[i1] = a * s + b * c;
            }
        }
    }
}

/* ----------------------------------------------------------------- GEMV/GEMM
 * GGUF layout (weights [N][K], K contiguous): tests/forward_parity_toy.rs:30-43,
 * device form cuda/kernels.cu:5037-5052. C[m][n] = sum_k A[m][k] * W[n*K + k]. */
ORC_API void orc_gemm_f32xf16_gguf(const float* A, const uint16_t* W, float* C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        const uint16_t* wr = W + (size_t)n * (size_t)K;
        for (int m = 0; m < M; ++m) {
            const float* a = A + (size_t)m * (size_t)K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += a[k] * orc_f16_to_f32(wr[k]);
            C[(size_t)m * (size_t)N + n] = acc;
        }
    }
}

/* Row-major B [K][N]: tests/gemm_f16xf16_f32.rs:26-38 (A f16) and
 * tests/gemm_mixed.rs:63-102 (A f32); device forms cuda/kernels.cu:4999-5032. */
ORC_API void orc_gemm_f16xf16_rowmajor(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k)
                acc += orc_f16_to_f32(A[(size_t)m * K + k]) * orc_f16_to_f32(B[(size_t)k * N + n]);
            C[(size_t)m * N + n] = acc;
        }
    }
}

ORC_API void orc_gemm_f32xf16_rowmajor(const float* A, const uint16_t* B, float* C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += A[(size_t)m * K + k] * orc_f16_to_f32(B[(size_t)k * N + n]);
            C[(size_t)m * N + n] = acc;
        }
    }
}

/* f16 storage / f32 compute / f16 result: cuda/kernels.cu:4981-4996. */
ORC_API void orc_gemm_f16_storage(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K) {
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k)
                acc += orc_f16_to_f32(A[(size_t)m * K + k]) * orc_f16_to_f32(B[(size_t)k * N + n]);
            C[(size_t)m * N + n] = orc_f32_to_f16(acc);
        }
}

/* ---------------------------------------------------------------------- Q8_0
 * 34-byte blocks {f16 d; int8 qs[32]}, value = d * q:
 * src/infer/embeddings.rs:80-140, cuda/kernels.cu:856-867. */
ORC_API void orc_q80_to_f32(const uint8_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        const uint8_t* blk = in + (i / 32) * 34;
        const uint16_t dbits = (uint16_t)(blk[0] | ((uint16_t)blk[1] << 8));
        const float d = orc_f16_to_f32(dbits);
        out[i] = d * (float)(int8_t)blk[2 + (i % 32)];
    }
}

/* The oracle-side quantiser used to make synthetic Q8_0 weights (the reference
 * defines only the dequant side): d = f16(max|w|/127), q = clamp(rint(w/d)). */
ORC_API void orc_q80_quantize(const float* in, uint8_t* out, size_t n) {
    const size_t blocks = n / 32;
    for (size_t b = 0; b < blocks; ++b) {
        const float* w = in + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(w[i]));
        const uint16_t dbits = orc_f32_to_f16(amax / 127.0f);
        const float d = orc_f16_to_f32(dbits);
        uint8_t* blk = out + b * 34;
        blk[0] = (uint8_t)(dbits & 0xff);
        blk[1] = (uint8_t)(dbits >> 8);
        for (int i = 0; i < 32; ++i) {
            int q = d > 0.0f ? (int)lrintf(w[i] / d) : 0;
            if (q > 127) q = 127;
            if (q < -127) q = -127;
            blk[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}

/* GGUF-layout GEMM over Q8_0 rows: the composition of q80_to_f32
 * (kernels.cu:856-867) with the GGUF GEMM (kernels.cu:5037-5052):
 * C[m][n] = sum_k A[m][k] * (d[n][k/32] * q[n][k]). K must be a multiple of 32. */
ORC_API void orc_gemm_f32xq80_gguf(const float* A, const uint8_t* W, float* C, int M, int N, int K) {
    const size_t row_bytes = (size_t)(K / 32) * 34;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        const uint8_t* wr = W + (size_t)n * row_bytes;
        for (int m = 0; m < M; ++m) {
            const float* a = A + (size_t)m * (size_t)K;
            float acc = 0.0f;
            for (int kb = 0; kb < K / 32; ++kb) {
                const uint8_t* blk = wr + (size_t)kb * 34;
                const float d = orc_f16_to_f32((uint16_t)(blk[0] | ((uint16_t)blk[1] << 8)));
                for (int i = 0; i < 32; ++i) acc += a[kb * 32 + i] * (d * (float)(int8_t)blk[2 + i]);
            }
            C[(size_t)m * (size_t)N + n] = acc;
        }
    }
}

/* ------------------------------------------------------- SwiGLU and residual
 * tests/forward_parity_toy.rs:56-58; cuda/kernels.cu:880-891, 869-878. */
ORC_API void orc_swiglu(const float* gate, const float* up, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        const float g = gate[i];
        out[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

ORC_API void orc_residual_add(const float* a, const float* b, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

/* ----------------------------------------------------- dense decode attention
 * The reference's host attention, src/cuda.rs:4561-4628 (three passes, f32,
 * sequential sums over d then t, exp(s - max), divide by denom, denom==0 -> 1),
 * with the GQA head mapping of tests/attention_parity_cuda_grid.rs:1415-1469
 * (q head h reads kv head h / (Hq/Hkv)).
 *
 * K/V are f16 in the reference's logical cache layout [token][kv_head][d]
 * (cuda/kernels.cu:5304-5312) for ONE sequence; token t starts at
 * t * kv_heads * head_dim. q, out: [q_heads * head_dim] f32. */
static void attention_one_head(const uint16_t* K, const uint16_t* V, const float* qh, float* outh,
                               const uint32_t* tokens, size_t n_tok, size_t kvh, size_t kv_heads,
                               size_t head_dim, float inv_sqrt, float* scores) {
    const size_t ept = kv_heads * head_dim;
    float max_s = -INFINITY;
    for (size_t i = 0; i < n_tok; ++i) {
        const size_t t = tokens ? tokens[i] : i;
        const uint16_t* k = K + t * ept + kvh * head_dim;
        float dot = 0.0f;
        for (size_t d = 0; d < head_dim; ++d) dot += qh[d] * orc_f16_to_f32(k[d]);
        const float s = dot * inv_sqrt;
        scores[i] = s;
        if (s > max_s) max_s = s;
    }
    float denom = 0.0f;
    for (size_t i = 0; i < n_tok; ++i) {
        const float e = expf(scores[i] - max_s);
        scores[i] = e;
        denom += e;
    }
    if (denom == 0.0f) denom = 1.0f;
    for (size_t d = 0; d < head_dim; ++d) {
        float acc = 0.0f;
        for (size_t i = 0; i < n_tok; ++i) {
            const size_t t = tokens ? tokens[i] : i;
            acc += (scores[i] / denom) * orc_f16_to_f32(V[t * ept + kvh * head_dim + d]);
        }
        outh[d] = acc;
    }
}

ORC_API int orc_attention_gqa(const uint16_t* K, const uint16_t* V, const float* q, float* out,
                              uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t seq_len) {
    if (kv_heads == 0 || q_heads % kv_heads != 0 || seq_len == 0) return -1;
    const uint32_t group = q_heads / kv_heads;
    const float inv_sqrt = 1.0f / sqrtf((float)head_dim);
    int err = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < (int)q_heads; ++h) {
        float* scores = (float*)malloc((size_t)seq_len * sizeof(float));
        if (!scores) { err = -2; continue; }
        attention_one_head(K, V, q + (size_t)h * head_dim, out + (size_t)h * head_dim, NULL, seq_len,
                           (size_t)h / group, kv_heads, head_dim, inv_sqrt, scores);
        free(scores);
    }
    return err;
}

/* Batched variable-length decode == per-sequence attention for every batch row
 * (tests/attention_batched_varlen.rs:200-221). K/V hold all sequence slots:
 * [slot][max_seq_len][kv_heads][d]; q/out packed [batch][q_heads][d]. */
ORC_API int orc_attention_gqa_batched(const uint16_t* K, const uint16_t* V, const uint32_t* seq_ids,
                                      const uint32_t* seq_lens, uint32_t batch, const float* q, float* out,
                                      uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                      uint32_t max_seq_len) {
    if (kv_heads == 0 || q_heads % kv_heads != 0) return -1;
    const uint32_t group = q_heads / kv_heads;
    const float inv_sqrt = 1.0f / sqrtf((float)head_dim);
    const size_t slot_elems = (size_t)max_seq_len * kv_heads * head_dim;
    int err = 0;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int b = 0; b < (int)batch; ++b) {
        for (int h = 0; h < (int)q_heads; ++h) {
            const uint32_t len = seq_lens[b];
            if (len == 0 || len > max_seq_len) { err = -3; continue; }
            float* scores = (float*)malloc((size_t)len * sizeof(float));
            if (!scores) { err = -2; continue; }
            const size_t off = (size_t)seq_ids[b] * slot_elems;
            attention_one_head(K + off, V + off, q + ((size_t)b * q_heads + h) * head_dim,
                               out + ((size_t)b * q_heads + h) * head_dim, NULL, len, (size_t)h / group,
                               kv_heads, head_dim, inv_sqrt, scores);
            free(scores);
        }
    }
    return err;
}

/* --------------------------------------------------------------- q4 V format
 * cuda/kernels.cu:2254-2311: per (token, kv head) scale = max|v|/7 (1/7 when
 * all-zero) over the f16-rounded V; q = clamp(lrintf(v/scale), -7, 7); byte =
 * (q[2p] & 15) | (q[2p+1] & 15) << 4. Dequantised value (kernels.cu:2260-2264,
 * 3085-3086) = f16(nibble * scale). `v` is one head: head_dim f16 values. */
ORC_API float orc_q4_quantize_head(const uint16_t* v, uint8_t* packed, uint32_t head_dim) {
    float max_v = 0.0f;
    for (uint32_t d = 0; d < head_dim; ++d) max_v = fmaxf(max_v, fabsf(orc_f16_to_f32(v[d])));
    const float scale = max_v > 0.0f ? max_v / 7.0f : 1.0f / 7.0f;
    for (uint32_t p = 0; p < head_dim / 2; ++p) {
        int qa = (int)lrintf(orc_f16_to_f32(v[2 * p]) / scale);
        int qb = (int)lrintf(orc_f16_to_f32(v[2 * p + 1]) / scale);
        qa = qa < -7 ? -7 : (qa > 7 ? 7 : qa);
        qb = qb < -7 ? -7 : (qb > 7 ? 7 : qb);
        packed[p] = (uint8_t)((qa & 0x0f) | ((qb & 0x0f) << 4));
    }
    return scale;
}

ORC_API float orc_q4_dequant(uint8_t packed, uint32_t lane, float scale) {
    const uint8_t nib = lane == 0 ? (packed & 0x0f) : ((packed >> 4) & 0x0f);
    const int sv = nib >= 8 ? (int)nib - 16 : (int)nib;
    return orc_f16_to_f32(orc_f32_to_f16((float)sv * scale));
}

/* --------------------------------------------- block scoring + top-k selection
 * Device algorithm cuda/kernels.cu:2861-2930 (per q head): for each old block b,
 * score_b = (sum_{t in b} q . K_t / len_b) * inv_sqrt, kept in a list of top_n
 * by insertion with strict '>' (ties keep the earlier = lower block index; NaN
 * and scores <= -1e30 are never inserted); host form kernels.cu:6526-6600.
 *
 * Two score forms are produced: `scores_f32` reproduces the device's f32 order
 * (thread d accumulates over tokens, then a 128-wide pairwise tree:
 * kernels.cu:2896-2909), `scores_f64` is the exact-arithmetic value used for the
 * tie rule of the parity tests.
 *
 * old_k: f16 [old_len][kv_heads][d] for one sequence. q: one q head [d].
 * out_blocks/out_scores: top_n entries in descending score order. */
ORC_API uint32_t orc_block_select_head(const uint16_t* old_k, const float* qh, uint32_t kvh, uint32_t kv_heads,
                                       uint32_t head_dim, uint32_t old_len, uint32_t block_size,
                                       uint32_t top_blocks, uint32_t* out_blocks, float* out_scores,
                                       float* scores_f32, double* scores_f64) {
    const uint32_t nb = old_len == 0 ? 0 : (old_len + block_size - 1) / block_size;
    const uint32_t top_n = top_blocks < nb ? top_blocks : nb;
    const size_t ept = (size_t)kv_heads * head_dim;
    const float inv_sqrt = head_dim == 64u ? 0.125f : (head_dim == 128u ? 0.08838834764831845f
                                                                          : 1.0f / sqrtf((float)head_dim));
    float sel_scores[64];
    uint32_t sel_blocks[64];
    for (int i = 0; i < 64; ++i) { sel_scores[i] = -1e30f; sel_blocks[i] = 0xffffffffu; }
    float lanes[128];
    for (uint32_t b = 0; b < nb; ++b) {
        const uint32_t t0 = b * block_size;
        const uint32_t t1 = t0 + block_size < old_len ? t0 + block_size : old_len;
        double exact = 0.0;
        for (int i = 0; i < 128; ++i) lanes[i] = 0.0f;
        for (uint32_t t = t0; t < t1; ++t) {
            const uint16_t* k = old_k + (size_t)t * ept + (size_t)kvh * head_dim;
            for (uint32_t d = 0; d < head_dim; ++d) {
                const float kf = orc_f16_to_f32(k[d]);
                lanes[d % 128] += qh[d] * kf;
                exact += (double)qh[d] * (double)kf;
            }
        }
        for (int stride = 64; stride > 0; stride >>= 1)
            for (int i = 0; i < stride; ++i) lanes[i] += lanes[i + stride];
        const float block_len = (float)(t1 - t0);
        const float score = (lanes[0] / block_len) * inv_sqrt;
        if (scores_f32) scores_f32[b] = score;
        if (scores_f64) scores_f64[b] = exact / (double)(t1 - t0) * (double)inv_sqrt;
        uint32_t insert = top_n;
        for (uint32_t i = 0; i < top_n; ++i) {
            if (score > sel_scores[i]) { insert = i; break; }
        }
        if (insert < top_n) {
            for (uint32_t j = top_n - 1; j > insert; --j) {
                sel_scores[j] = sel_scores[j - 1];
                sel_blocks[j] = sel_blocks[j - 1];
            }
            sel_scores[insert] = score;
            sel_blocks[insert] = b;
        }
    }
    uint32_t count = 0;
    for (uint32_t i = 0; i < top_n; ++i) {
        if (sel_blocks[i] == 0xffffffffu) continue;
        out_blocks[count] = sel_blocks[i];
        if (out_scores) out_scores[count] = sel_scores[i];
        ++count;
    }
    return count;
}

/* ------------------------------------- compressed (FP16-K / q4-V) attention
 * cuda/kernels.cu:2832-3096 with the default policy (top-k, score order).
 * Logical state of one sequence, reference layouts (kernels.cu:5357-5385):
 *   old_k   f16 [old tokens][kv_heads][d]      (token index = absolute position)
 *   q4_v    u8  [old tokens][kv_heads][d/2], q4_scale f32 [old tokens][kv_heads]
 *   recent_k/recent_v f16 ring [recent_window][kv_heads][d], token t at t % R
 * Token list per q head = tokens of the selected blocks (descending score), then
 * the recent tokens [old_len, seq_len); three-pass softmax as the dense path.
 * selected_out (optional): [q_heads][64] block indices, 0xffffffff padded;
 * selected_count_out [q_heads]; union_tokens_out (optional): number of distinct
 * (kv head, old token) pairs touched, the `U` of the traffic model. */
ORC_API int orc_attention_compressed(const uint16_t* old_k, const uint8_t* q4_v, const float* q4_scale,
                                     const uint16_t* recent_k, const uint16_t* recent_v, const float* q,
                                     float* out, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                     uint32_t seq_len, uint32_t recent_window, uint32_t block_size,
                                     uint32_t top_blocks, uint32_t* selected_out,
                                     uint32_t* selected_count_out, uint64_t* union_tokens_out) {
    if (kv_heads == 0 || q_heads % kv_heads != 0 || seq_len == 0) return -1;
    if (recent_window == 0 || block_size == 0 || top_blocks == 0 || top_blocks > 64) return -6;
    const uint32_t group = q_heads / kv_heads;
    const uint32_t old_len = seq_len > recent_window ? seq_len - recent_window : 0;
    const uint32_t nb = old_len == 0 ? 0 : (old_len + block_size - 1) / block_size;
    const size_t ept = (size_t)kv_heads * head_dim;
    const size_t ppt = (size_t)kv_heads * (head_dim / 2);
    const float inv_sqrt = head_dim == 64u ? 0.125f : (head_dim == 128u ? 0.08838834764831845f
                                                                          : 1.0f / sqrtf((float)head_dim));
    uint8_t* touched = union_tokens_out ? (uint8_t*)calloc((size_t)kv_heads * (nb ? nb : 1), 1) : NULL;
    int err = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < (int)q_heads; ++h) {
        const uint32_t kvh = (uint32_t)h / group;
        const float* qh = q + (size_t)h * head_dim;
        uint32_t blocks[64];
        const uint32_t cnt = orc_block_select_head(old_k, qh, kvh, kv_heads, head_dim, old_len, block_size,
                                                   top_blocks, blocks, NULL, NULL, NULL);
        if (selected_out) {
            for (uint32_t i = 0; i < 64; ++i) selected_out[(size_t)h * 64 + i] = i < cnt ? blocks[i] : 0xffffffffu;
        }
        if (selected_count_out) selected_count_out[h] = cnt;
        if (touched) {
            for (uint32_t i = 0; i < cnt; ++i) {
#pragma omp atomic write
                touched[(size_t)kvh * nb + blocks[i]] = 1;
            }
        }
        const size_t cap = (size_t)cnt * block_size + recent_window;
        uint32_t* toks = (uint32_t*)malloc(cap * sizeof(uint32_t));
        float* scores = (float*)malloc(cap * sizeof(float));
        if (!toks || !scores) { err = -2; free(toks); free(scores); continue; }
        size_t n = 0;
        for (uint32_t i = 0; i < cnt; ++i) {
            const uint32_t t0 = blocks[i] * block_size;
            const uint32_t t1 = t0 + block_size < old_len ? t0 + block_size : old_len;
            for (uint32_t t = t0; t < t1; ++t) toks[n++] = t;
        }
        for (uint32_t t = old_len; t < seq_len; ++t) toks[n++] = t;
        float max_s = -1e30f;
        for (size_t i = 0; i < n; ++i) {
            const uint32_t t = toks[i];
            const uint16_t* k = t < old_len ? old_k + (size_t)t * ept + (size_t)kvh * head_dim
                                            : recent_k + (size_t)(t % recent_window) * ept + (size_t)kvh * head_dim;
            float dot = 0.0f;
            for (uint32_t d = 0; d < head_dim; ++d) dot += qh[d] * orc_f16_to_f32(k[d]);
            scores[i] = dot * inv_sqrt;
            if (scores[i] > max_s) max_s = scores[i];
        }
        float denom = 0.0f;
        for (size_t i = 0; i < n; ++i) denom += expf(scores[i] - max_s);
        denom = denom > 0.0f ? denom : 1.0f;
        float* outh = out + (size_t)h * head_dim;
        for (uint32_t d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (size_t i = 0; i < n; ++i) {
                const uint32_t t = toks[i];
                const float p = expf(scores[i] - max_s) / denom;
                float v;
                if (t < old_len) {
                    const uint8_t byte = q4_v[(size_t)t * ppt + (size_t)kvh * (head_dim / 2) + d / 2];
                    v = orc_q4_dequant(byte, d & 1u, q4_scale[(size_t)t * kv_heads + kvh]);
                } else {
                    v = orc_f16_to_f32(recent_v[(size_t)(t % recent_window) * ept + (size_t)kvh * head_dim + d]);
                }
                acc += p * v;
            }
            outh[d] = acc;
        }
        free(toks);
        free(scores);
    }
    if (touched) {
        uint64_t u = 0;
        for (uint32_t kvh = 0; kvh < kv_heads; ++kvh)
            for (uint32_t b = 0; b < nb; ++b)
                if (touched[(size_t)kvh * nb + b]) {
                    const uint32_t t0 = b * block_size;
                    const uint32_t t1 = t0 + block_size < old_len ? t0 + block_size : old_len;
                    u += t1 - t0;
                }
        *union_tokens_out = u;
        free(touched);
    }
    return err;
}

/* The dense-FP16-backed form of the same selection (cuda/kernels.cu:1825-1983,
 * launcher 4025-4070): K and V both f16 in the dense layout [token][kv_head][d];
 * token list and softmax exactly as above. */
ORC_API int orc_attention_block_select_dense(const uint16_t* K, const uint16_t* V, const float* q, float* out,
                                             uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                             uint32_t seq_len, uint32_t recent_window, uint32_t block_size,
                                             uint32_t top_blocks) {
    if (kv_heads == 0 || q_heads % kv_heads != 0 || seq_len == 0) return -1;
    if (recent_window == 0 || block_size == 0 || top_blocks == 0 || top_blocks > 64) return -6;
    const uint32_t group = q_heads / kv_heads;
    const uint32_t old_len = seq_len > recent_window ? seq_len - recent_window : 0;
    const float inv_sqrt = head_dim == 64u ? 0.125f : (head_dim == 128u ? 0.08838834764831845f
                                                                          : 1.0f / sqrtf((float)head_dim));
    int err = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < (int)q_heads; ++h) {
        const uint32_t kvh = (uint32_t)h / group;
        uint32_t blocks[64];
        const uint32_t cnt = orc_block_select_head(K, q + (size_t)h * head_dim, kvh, kv_heads, head_dim, old_len,
                                                   block_size, top_blocks, blocks, NULL, NULL, NULL);
        const size_t cap = (size_t)cnt * block_size + recent_window;
        uint32_t* toks = (uint32_t*)malloc(cap * sizeof(uint32_t));
        float* scores = (float*)malloc(cap * sizeof(float));
        if (!toks || !scores) { err = -2; free(toks); free(scores); continue; }
        size_t n = 0;
        for (uint32_t i = 0; i < cnt; ++i) {
            const uint32_t t0 = blocks[i] * block_size;
            const uint32_t t1 = t0 + block_size < old_len ? t0 + block_size : old_len;
            for (uint32_t t = t0; t < t1; ++t) toks[n++] = t;
        }
        for (uint32_t t = old_len; t < seq_len; ++t) toks[n++] = t;
        attention_one_head(K, V, q + (size_t)h * head_dim, out + (size_t)h * head_dim, toks, n, kvh, kv_heads,
                           head_dim, inv_sqrt, scores);
        free(toks);
        free(scores);
    }
    return err;
}

/* -------------------------------------------------------------- split-K merge
 * Partial triples (m, l, o[d]) per q head from P ranks (o unnormalised:
 * o_r = sum_t exp(s_t - m_r) v_t, l_r = sum_t exp(s_t - m_r)); merged
 * out = sum_r e^{m_r-M} o_r / sum_r e^{m_r-M} l_r, M = max_r m_r. Ranks with
 * l_r == 0 (no tokens) carry m_r = -inf and contribute nothing.
 * This has no reference counterpart (the reference is single-GPU); it is the
 * algebraic identity the multi-GPU tests check against orc_attention_gqa. */
ORC_API void orc_merge_partials(const float* m, const float* l, const float* o, float* out, uint32_t parts,
                                uint32_t heads, uint32_t head_dim) {
    for (uint32_t h = 0; h < heads; ++h) {
        float M = -INFINITY;
        for (uint32_t r = 0; r < parts; ++r)
            if (l[(size_t)r * heads + h] > 0.0f && m[(size_t)r * heads + h] > M) M = m[(size_t)r * heads + h];
        float L = 0.0f;
        for (uint32_t r = 0; r < parts; ++r)
            if (l[(size_t)r * heads + h] > 0.0f) L += expf(m[(size_t)r * heads + h] - M) * l[(size_t)r * heads + h];
        if (!(L > 0.0f)) L = 1.0f;
        for (uint32_t d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (uint32_t r = 0; r < parts; ++r)
                if (l[(size_t)r * heads + h] > 0.0f)
                    acc += expf(m[(size_t)r * heads + h] - M) * o[((size_t)r * heads + h) * head_dim + d];
            out[(size_t)h * head_dim + d] = acc / L;
        }
    }
}

/* ---------------------------------------------------------- whole decode layer
 * Op order of src/infer/forward.rs:247-667 (see tests/forward_parity_toy.rs:309-386):
 *   xn = rmsnorm(x, w_attn_norm); q,k,v = xn.Wq/Wk/Wv (+ f32 biases, forward.rs:124-163)
 *   q = rope(q, pos); K[pos] = f16(rope(k, pos)); V[pos] = f16(v)      (kernels.cu:5624-5676)
 *   att = attention over tokens [0, pos]; y = att.Wo; x1 = x + y
 *   x1n = rmsnorm(x1, w_ffn_norm); hid = silu(x1n.Wg) * (x1n.Wu); out = x1 + hid.Wd
 * Weights are GGUF layout [N][K]; attention weights f16; FFN weights f16
 * (ffn_q80 == 0) or Q8_0 rows (ffn_q80 == 1). K/V: f16 dense cache of ONE
 * sequence [max_seq][kv_heads][d], updated in place at `pos`. */
typedef struct {
    uint32_t hidden, q_heads, kv_heads, head_dim, ffn, ffn_q80, rope_layout;
    float eps, rope_base, rope_scale;
} orc_layer_cfg;

ORC_API int orc_decode_layer(const orc_layer_cfg* c, const float* x, float* out, const float* w_attn_norm,
                             const uint16_t* wq, const uint16_t* wk, const uint16_t* wv, const uint16_t* wo,
                             const float* bq, const float* bk, const float* bv, const float* w_ffn_norm,
                             const void* wg, const void* wu, const void* wd, uint16_t* K, uint16_t* V,
                             uint32_t pos, float* dbg_q, float* dbg_att) {
    const uint32_t H = c->hidden, QD = c->q_heads * c->head_dim, KD = c->kv_heads * c->head_dim, F = c->ffn;
    float* xn = (float*)malloc(sizeof(float) * H);
    float* q = (float*)malloc(sizeof(float) * QD);
    float* k = (float*)malloc(sizeof(float) * KD);
    float* v = (float*)malloc(sizeof(float) * KD);
    float* att = (float*)malloc(sizeof(float) * QD);
    float* y = (float*)malloc(sizeof(float) * H);
    float* x1 = (float*)malloc(sizeof(float) * H);
    float* x1n = (float*)malloc(sizeof(float) * H);
    float* gate = (float*)malloc(sizeof(float) * F);
    float* up = (float*)malloc(sizeof(float) * F);
    float* hid = (float*)malloc(sizeof(float) * F);
    int rc = 0;
    if (!xn || !q || !k || !v || !att || !y || !x1 || !x1n || !gate || !up || !hid) { rc = -2; goto done; }
    orc_rms_norm(x, w_attn_norm, xn, 1, H, c->eps);
    orc_gemm_f32xf16_gguf(xn, wq, q, 1, (int)QD, (int)H);
    orc_gemm_f32xf16_gguf(xn, wk, k, 1, (int)KD, (int)H);
    orc_gemm_f32xf16_gguf(xn, wv, v, 1, (int)KD, (int)H);
    if (bq) orc_residual_add(q, bq, q, QD);
    if (bk) orc_residual_add(k, bk, k, KD);
    if (bv) orc_residual_add(v, bv, v, KD);
    orc_rope(q, 1, c->q_heads, c->head_dim, pos, c->rope_base, c->rope_scale, c->rope_layout);
    orc_rope(k, 1, c->kv_heads, c->head_dim, pos, c->rope_base, c->rope_scale, c->rope_layout);
    orc_f32_to_f16_array(k, K + (size_t)pos * KD, KD);
    orc_f32_to_f16_array(v, V + (size_t)pos * KD, KD);
    if (dbg_q) memcpy(dbg_q, q, sizeof(float) * QD);
    rc = orc_attention_gqa(K, V, q, att, c->q_heads, c->kv_heads, c->head_dim, pos + 1);
    if (rc != 0) goto done;
    if (dbg_att) memcpy(dbg_att, att, sizeof(float) * QD);
    orc_gemm_f32xf16_gguf(att, wo, y, 1, (int)H, (int)QD);
    orc_residual_add(x, y, x1, H);
    orc_rms_norm(x1, w_ffn_norm, x1n, 1, H, c->eps);
    if (c->ffn_q80) {
        orc_gemm_f32xq80_gguf(x1n, (const uint8_t*)wg, gate, 1, (int)F, (int)H);
        orc_gemm_f32xq80_gguf(x1n, (const uint8_t*)wu, up, 1, (int)F, (int)H);
    } else {
        orc_gemm_f32xf16_gguf(x1n, (const uint16_t*)wg, gate, 1, (int)F, (int)H);
        orc_gemm_f32xf16_gguf(x1n, (const uint16_t*)wu, up, 1, (int)F, (int)H);
    }
    orc_swiglu(gate, up, hid, F);
    if (c->ffn_q80) orc_gemm_f32xq80_gguf(hid, (const uint8_t*)wd, y, 1, (int)H, (int)F);
    else orc_gemm_f32xf16_gguf(hid, (const uint16_t*)wd, y, 1, (int)H, (int)F);
    orc_residual_add(x1, y, out, H);
done:
    free(xn); free(q); free(k); free(v); free(att); free(y); free(x1); free(x1n); free(gate); free(up); free(hid);
    return rc;
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Packed variable-length causal prefill attention, f32 throughout: cuda/kernels.cu:3749-3835 (three passes: scores of
 * kv rows 0 .. kv_len - q_len + i, their maximum, exp / sum, then the weighted V sum with p = exp(s - max) / denom). */
ORC_API int orc_attention_prefill_varlen(const float* q, const float* k, const float* v, const uint32_t* q_off,
                                 const uint32_t* kv_off, const uint32_t* q_lens, const uint32_t* kv_lens, uint32_t batch,
                                 uint32_t q_heads, uint32_t kv_heads, uint32_t hd, float* out) {
    if (!q || !k || !v || !out || kv_heads == 0 || q_heads % kv_heads != 0) return -1;
    const uint32_t group = q_heads / kv_heads;
    const float inv_sqrt = hd == 64u ? 0.125f : (hd == 128u ? 0.08838834764831845f : 1.0f / sqrtf((float)hd));
    for (uint32_t b = 0; b < batch; ++b) {
        const uint32_t ql = q_lens[b], kl = kv_lens[b];
        if (ql == 0 || kl == 0 || ql > kl) return -8;
#pragma omp parallel for collapse(2) schedule(dynamic)
        for (uint32_t i = 0; i < ql; ++i) {
            for (uint32_t h = 0; h < q_heads; ++h) {
                const uint32_t end = kl - ql + i, kvh = h / group;
                const float* qh = q + ((size_t)(q_off[b] + i) * q_heads + h) * hd;
                float* scores = (float*)malloc((size_t)(end + 1) * sizeof(float));
                float mx = -1e30f;
                for (uint32_t t = 0; t <= end; ++t) {
                    const float* kh = k + ((size_t)(kv_off[b] + t) * kv_heads + kvh) * hd;
                    float dot = 0.0f;
                    for (uint32_t d = 0; d < hd; ++d) dot += qh[d] * kh[d];
                    scores[t] = dot * inv_sqrt;
                    if (scores[t] > mx) mx = scores[t];
                }
                float denom = 0.0f;
                for (uint32_t t = 0; t <= end; ++t) denom += expf(scores[t] - mx);
                if (!(denom > 0.0f)) denom = 1.0f;
                float* oh = out + ((size_t)(q_off[b] + i) * q_heads + h) * hd;
                for (uint32_t d = 0; d < hd; ++d) {
                    float acc = 0.0f;
                    for (uint32_t t = 0; t <= end; ++t) {
                        const float* vh = v + ((size_t)(kv_off[b] + t) * kv_heads + kvh) * hd;
                        acc += (expf(scores[t] - mx) / denom) * vh[d];
                    }
                    oh[d] = acc;
                }
                free(scores);
            }
        }
    }
    return 0;
}

