"""Generates golden output vectors by running a library that exports the m40llm C ABI.

    python tests/golden/make_golden.py --lib ref  --out tests/golden/ref_b200.npz   # the reference's own
                                                                                     # cuda/kernels.cu, built
                                                                                     # unmodified for sm_100a
                                                                                     # by `make -C oracle ref`
    python tests/golden/make_golden.py --lib mine --out /tmp/mine.npz               # this repo's library

Needs a CUDA device. Inputs come from tests/golden/cases.py (seeded); only outputs are written.
The committed ref_b200.npz was produced with `--lib ref` on an NVIDIA B200.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
import cases  # noqa: E402
import helpers  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib", choices=["ref", "mine"], required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--only", default="", help="comma-separated case-name prefixes to generate (default: everything)")
    ap.add_argument("--merge-into", default="", help="existing .npz whose arrays are kept and extended by this run")
    args = ap.parse_args()
    only = [x for x in args.only.split(",") if x]
    want = lambda name: not only or any(name.startswith(x) for x in only)
    pkg = helpers.load_package()
    if args.lib == "ref":
        dll = helpers.load_reference_lib(pkg)
        assert dll is not None, "oracle/_ref/libm40llm_ref.so is missing: run `make -C oracle ref`"
    else:
        dll = pkg.native.lib()
    nat = helpers.Native(dll)
    L, ctx = nat.lib, nat.ctx
    out = {}
    p = lambda a: a.ctypes.data_as(C.c_void_p)

    for name, (rows, dim) in cases.NORM_CASES.items():
        if not want(name):
            continue
        x, w = cases.norm_inputs(name)
        dx, dw, dy = nat.buf(x), nat.buf(w), nat.buf(x.nbytes)
        assert L.m40llm_rms_norm_f32_async(ctx, dx.ptr, dy.ptr, rows, dim, 1e-5) == 0
        nat.sync(1)
        out[name + "/plain"] = dy.download(np.float32, x.shape)
        assert L.m40llm_rms_norm_f32_weighted_async(ctx, dx.ptr, dw.ptr, dy.ptr, rows, dim, 1e-5, 1) == 0
        nat.sync(1)
        out[name + "/weighted"] = dy.download(np.float32, x.shape)
        nat.free_all()

    for name, (rows, heads, hd, past, base, layout) in cases.ROPE_CASES.items():
        if not want(name):
            continue
        x = cases.rope_inputs(name)
        dx = nat.buf(x)
        assert L.m40llm_rope_f32_inplace_layout_async(ctx, dx.ptr, rows, heads, hd, past, base, 1.0, layout) == 0
        nat.sync(1)
        out[name] = dx.download(np.float32, x.shape)
        nat.free_all()

    for name, (M, N, K) in cases.GEMM_CASES.items():
        if not want(name):
            continue
        a, w = cases.gemm_inputs(name)
        b = np.ascontiguousarray(w.T)
        da, da16, dw, db, dc = nat.buf(a), nat.buf(a.astype(np.float16)), nat.buf(w), nat.buf(b), nat.buf(M * N * 4)
        assert L.m40llm_gemm_f32xf16_gguf_f32(ctx, da.ptr, dw.ptr, dc.ptr, M, N, K) == 0
        out[name + "/gguf"] = dc.download(np.float32, (M, N))
        assert L.m40llm_gemm_f32xf16_f32(ctx, da.ptr, db.ptr, dc.ptr, M, N, K) == 0
        out[name + "/f32xf16"] = dc.download(np.float32, (M, N))
        assert L.m40llm_gemm_f16xf16_f32(ctx, da16.ptr, db.ptr, dc.ptr, M, N, K) == 0
        out[name + "/f16xf16"] = dc.download(np.float32, (M, N))
        nat.free_all()

    # elementwise + Q8_0 dequant
    r = cases.rng_for("elementwise")
    g = (r.standard_normal(5000) * 3).astype(np.float32)
    u = r.standard_normal(5000).astype(np.float32)
    dg, du, do = nat.buf(g), nat.buf(u), nat.buf(g.nbytes)
    assert L.m40llm_swiglu_f32_async(ctx, dg.ptr, du.ptr, do.ptr, g.size) == 0
    nat.sync(1)
    out["swiglu"] = do.download(np.float32, g.shape)
    from oracle import oracle as O
    q80 = O.q80_quantize((r.standard_normal((4, 256)) * 0.02).astype(np.float32))
    dq80, dd = nat.buf(q80), nat.buf(4 * 256 * 4)
    assert L.m40llm_q80_to_f32(ctx, dq80.ptr, dd.ptr, 4 * 256) == 0
    out["q80_to_f32"] = dd.download(np.float32, (4, 256))
    nat.free_all()

    for name, (qh, kvh, hd, Ln) in cases.ATTN_CASES.items():
        if not want(name):
            continue
        k, v, q = cases.attn_inputs(name)
        kv = nat.kv_dense(Ln, 1, kvh, hd)
        # K through the fused RoPE append (theta 1e4, adjacent) so the cache content itself is a golden
        nat.kv_append_tokens(kv, 0, k, v, base=1e4, scale=1.0, layout=0)
        toks = cases.cache_sample_tokens(Ln)
        kk = np.empty((len(toks), kvh, hd), np.float16)
        vv = np.empty((len(toks), kvh, hd), np.float16)
        for i, t in enumerate(toks):
            assert L.m40llm_kvcache_debug_read_token(ctx, kv, 0, t, p(kk[i]), p(vv[i])) == 0
        out[name + "/k_cache"] = kk.view(np.uint16)
        out[name + "/v_cache"] = vv.view(np.uint16)
        dq, do = nat.buf(q), nat.buf(q.nbytes)
        assert L.m40llm_attention_last_token_f32_gqa_async(ctx, kv, 0, dq.ptr, qh, Ln, do.ptr) == 0
        nat.sync(1)
        out[name + "/out"] = do.download(np.float32, q.shape)
        if hd == 64:  # the reference's block-select-over-dense kernel is head_dim 64 only
            assert L.m40llm_attention_last_token_f32_gqa_block_select_exact_async(ctx, kv, 0, dq.ptr, qh, Ln, 16, 8, 4, do.ptr) == 0
            nat.sync(1)
            out[name + "/block_select_dense_R16_bs8_top4"] = do.download(np.float32, q.shape)
        L.m40llm_kvcache_destroy(kv)
        nat.free_all()

    for name, (qh, kvh, hd, lens) in cases.BATCH_CASES.items():
        if not want(name):
            continue
        ks, vs, q = cases.batch_inputs(name)
        kv = nat.kv_dense(max(lens), len(lens), kvh, hd)
        for b in range(len(lens)):
            nat.kv_append_tokens(kv, b, ks[b], vs[b], scale=0.0)
        dq, do = nat.buf(q), nat.buf(q.nbytes)
        dids, dlens = nat.buf(np.arange(len(lens), dtype=np.uint32)), nat.buf(np.array(lens, np.uint32))
        assert L.m40llm_attention_last_token_f32_gqa_batched(ctx, kv, dids.ptr, dlens.ptr, len(lens), dq.ptr, qh, do.ptr) == 0
        out[name + "/out"] = do.download(np.float32, q.shape)
        L.m40llm_kvcache_destroy(kv)
        nat.free_all()

    for name, (qh, kvh, hd, Ln, R, bs, top) in cases.Q4_CASES.items():
        if not want(name):
            continue
        k, v, q = cases.q4_inputs(name)
        kv = nat.kv_compressed(Ln, 1, kvh, hd, R, bs, top)
        nat.kv_append_tokens(kv, 0, k, v, scale=0.0)
        dq, do = nat.buf(q), nat.buf(q.nbytes)
        rc = L.m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async(
            ctx, kv, 0, dq.ptr, qh, Ln, R, bs, top, do.ptr)
        assert rc == 0, rc
        nat.sync(1)
        out[name + "/out"] = do.download(np.float32, q.shape)
        blocks = np.zeros(64, np.uint32); scores = np.zeros(64, np.float32); st = np.zeros(64, np.uint32); en = np.zeros(64, np.uint32)
        cnt, total = C.c_uint32(), C.c_uint32()
        rc = L.m40llm_kvcache_debug_select_old_blocks(ctx, kv, 0, dq.ptr, qh, Ln, R, bs, top, p(blocks), p(scores), p(st), p(en),
                                                      C.byref(cnt), 64, C.byref(total))
        assert rc == 0, rc
        out[name + "/head0_blocks"] = blocks[:cnt.value].copy()
        out[name + "/head0_scores"] = scores[:cnt.value].copy()
        out[name + "/total_blocks"] = np.array([total.value], np.uint32)
        L.m40llm_kvcache_destroy(kv)
        nat.free_all()

    for name, (qh, kvh, hd, pairs) in cases.PREFILL_CASES.items():
        if not want(name):
            continue
        q, k, v, qo, ko, ql, kl = cases.prefill_inputs(name)
        dq, dk, dv, do = nat.buf(q), nat.buf(k), nat.buf(v), nat.buf(q.nbytes)
        dqo, dko, dql, dkl = nat.buf(qo), nat.buf(ko), nat.buf(ql), nat.buf(kl)
        rc = L.m40llm_attention_prefill_f32_gqa_varlen(ctx, dq.ptr, dk.ptr, dv.ptr, dqo.ptr, dko.ptr, dql.ptr, dkl.ptr,
                                                       len(pairs), qh, kvh, hd, do.ptr)
        assert rc == 0, rc
        nat.sync(0)
        out[name + "/out"] = do.download(np.float32, q.shape)[cases.prefill_sample_rows(name)]
        nat.free_all()

    if args.merge_into and os.path.exists(args.merge_into):
        merged = dict(np.load(args.merge_into))
        merged.update(out)
        out = merged
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
