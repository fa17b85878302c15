"""Whole decode layer through the C ABI against the oracle's layer (op order of src/infer/forward.rs:247-667,
CPU form tests/forward_parity_toy.rs:309-386; the reference's toy-layer tolerance is 5e-3)."""
import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu


def make_weights(O, rng, H, qh, kvh, hd, F, q80, bias):
    w = {}
    for n, s in dict(wq=(qh * hd, H), wk=(kvh * hd, H), wv=(kvh * hd, H), wo=(H, qh * hd)).items():
        w[n] = (rng.standard_normal(s) * 0.02).astype(np.float16)
    for n, s in dict(wg=(F, H), wu=(F, H), wd=(H, F)).items():
        f = (rng.standard_normal(s) * 0.02).astype(np.float32)
        w[n] = O.q80_quantize(f) if q80 else f.astype(np.float16)
    w["attn_norm"] = (1 + 0.05 * rng.standard_normal(H)).astype(np.float32)
    w["ffn_norm"] = (1 + 0.05 * rng.standard_normal(H)).astype(np.float32)
    if bias:
        w["bq"] = (rng.standard_normal(qh * hd) * 0.02).astype(np.float32)
        w["bk"] = (rng.standard_normal(kvh * hd) * 0.02).astype(np.float32)
        w["bv"] = (rng.standard_normal(kvh * hd) * 0.02).astype(np.float32)
    return w


def device_layer(nat, kv, w, x_rows, seq_ids, positions, cfg, q80):
    """The layer as the fused entry points issue it: prologue, batched attention, Wo+residual, FFN+residual."""
    L, ctx = nat.lib, nat.ctx
    rows = x_rows.shape[0]
    H, qd, F = cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.ffn
    d = {n: nat.buf(a) for n, a in w.items()}
    dx, dq, datt, dx1, dx1n = nat.buf(x_rows), nat.buf(rows * qd * 4), nat.buf(rows * qd * 4), nat.buf(rows * H * 4), nat.buf(rows * H * 4)
    dhid, dout = nat.buf(rows * F * 4), nat.buf(rows * H * 4)
    dids, dpos = nat.buf(np.asarray(seq_ids, np.uint32)), nat.buf(np.asarray(positions, np.uint32))
    dlens = nat.buf(np.asarray(positions, np.uint32) + 1)
    g = lambda n: d[n].ptr if n in d else None
    rc = L.m40llm_qkv_rmsnorm_rope_append_async(ctx, kv, dx.ptr, d["attn_norm"].ptr, 1, cfg.eps, d["wq"].ptr, d["wk"].ptr,
                                                d["wv"].ptr, g("bq"), g("bk"), g("bv"), dids.ptr, dpos.ptr, rows, H,
                                                cfg.q_heads, cfg.rope_base, cfg.rope_scale, cfg.rope_layout, dq.ptr)
    assert rc == 0, rc
    assert L.m40llm_attention_last_token_f32_gqa_batched_async(ctx, kv, dids.ptr, dlens.ptr, rows, dq.ptr, cfg.q_heads, datt.ptr) == 0
    # y = att.Wo ; x1 = x + y   (decode stream throughout: no cross-stream waits needed)
    assert L.m40llm_gemm_f32xf16_gguf_f32_async(ctx, datt.ptr, d["wo"].ptr, dx1.ptr, rows, H, qd, 1) == 0
    assert L.m40llm_residual_add_f32_async(ctx, dx.ptr, dx1.ptr, dx1.ptr, rows * H) == 0
    assert L.m40llm_rms_norm_f32_weighted_async(ctx, dx1.ptr, d["ffn_norm"].ptr, dx1n.ptr, rows, H, cfg.eps, 1) == 0
    ffn = L.m40llm_ffn_swiglu_q80_f32_async if q80 else L.m40llm_ffn_swiglu_f16_f32_async
    assert ffn(ctx, dx1n.ptr, d["wg"].ptr, d["wu"].ptr, d["wd"].ptr, dx1.ptr, dhid.ptr, dout.ptr, rows, H, F, 1) == 0
    nat.sync(1)
    return (dout.download(np.float32, (rows, H)), dq.download(np.float32, (rows, qd)), datt.download(np.float32, (rows, qd)))


@pytest.mark.parametrize("H,qh,kvh,hd,F,q80,layout,bias,base,ctx_len", [
    (64, 4, 2, 16, 128, False, 0, False, 1e4, 5),        # toy layer
    (256, 8, 2, 64, 384, True, 0, False, 1e4, 40),       # q8 FFN, adjacent RoPE
    (2048, 32, 4, 64, 5632, False, 0, False, 1e4, 300),  # TinyLlama-shaped layer
    (2048, 16, 2, 128, 1024, False, 1, True, 1e6, 200),  # Qwen heads: NeoX RoPE + QKV bias
    (4096, 32, 8, 128, 14336, True, 0, False, 5e5, 600), # Llama-3-8B-shaped layer, Q8_0 FFN
])
def test_decode_layer_single_row(nat, O, H, qh, kvh, hd, F, q80, layout, bias, base, ctx_len):
    rng = np.random.default_rng(H + F)
    cfg = O.LayerCfg(H, qh, kvh, hd, F, 1 if q80 else 0, layout, 1e-5, base, 1.0)
    w = make_weights(O, rng, H, qh, kvh, hd, F, q80, bias)
    max_seq = ctx_len + 4
    K = np.zeros((max_seq, kvh, hd), np.float16)
    V = np.zeros((max_seq, kvh, hd), np.float16)
    K[:ctx_len] = rng.standard_normal((ctx_len, kvh, hd)).astype(np.float16)
    V[:ctx_len] = rng.standard_normal((ctx_len, kvh, hd)).astype(np.float16)
    kv = nat.kv_dense(max_seq, 1, kvh, hd)
    nat.kv_fill(kv, 0, K[:ctx_len], V[:ctx_len])
    x = rng.standard_normal(H).astype(np.float32)
    # two consecutive tokens (tests/forward_parity_toy.rs runs one and two tokens)
    for step in range(2):
        pos = ctx_len + step
        out, q_rot, att = device_layer(nat, kv, w, x[None, :], [0], [pos], cfg, q80)
        eout, eq, eatt = O.decode_layer(cfg, x, w, K, V, pos)
        assert_close(q_rot[0], eq, what=f"q after rope, step {step}")
        assert_close(att[0], eatt, what=f"attention, step {step}")
        assert_close(out[0], eout, what=f"layer output, step {step}")
        x = eout
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_decode_layer_batched_rows_and_compressed_append(nat, O):
    """Batched decode rows (src/infer/forward.rs:1729-2140): every row equals the single-row layer on its own
    sequence; the fused prologue also feeds a compressed cache (ring + eviction)."""
    rng = np.random.default_rng(77)
    H, qh, kvh, hd, F = 512, 8, 2, 64, 768
    cfg = O.LayerCfg(H, qh, kvh, hd, F, 1, 0, 1e-5, 1e4, 1.0)
    w = make_weights(O, rng, H, qh, kvh, hd, F, True, False)
    lens = [37, 5, 120, 64, 1]
    B, max_seq = len(lens), 128
    kv = nat.kv_dense(max_seq, B, kvh, hd)
    Ks = [np.zeros((max_seq, kvh, hd), np.float16) for _ in range(B)]
    Vs = [np.zeros((max_seq, kvh, hd), np.float16) for _ in range(B)]
    for b, n in enumerate(lens):
        Ks[b][:n - 1] = rng.standard_normal((n - 1, kvh, hd)).astype(np.float16)
        Vs[b][:n - 1] = rng.standard_normal((n - 1, kvh, hd)).astype(np.float16)
        if n > 1:
            nat.kv_fill(kv, b, Ks[b][:n - 1], Vs[b][:n - 1])
    x = rng.standard_normal((B, H)).astype(np.float32)
    out, q_rot, att = device_layer(nat, kv, w, x, list(range(B)), [n - 1 for n in lens], cfg, True)
    for b, n in enumerate(lens):
        eout, eq, eatt = O.decode_layer(cfg, x[b], w, Ks[b], Vs[b], n - 1)
        assert_close(att[b], eatt, what=f"row {b} attention")
        assert_close(out[b], eout, what=f"row {b} output")
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()
