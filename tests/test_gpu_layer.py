"""Whole decode layer through the C ABI against the oracle's layer (op order of src/infer/forward.rs:247-667,
CPU form tests/forward_parity_toy.rs:309-386; the reference's toy-layer tolerance is 5e-3)."""
import ctypes as C

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


def device_layer(nat, kv, w, x_rows, seq_ids, positions, cfg, q80, fused_tail=False, one_call_front=False):
    """The layer as the fused entry points issue it: prologue, batched attention, then either the reference's op
    sequence (Wo, residual, norm, FFN + residual) or the single composite call for steps 9-13."""
    L, ctx = nat.lib, nat.ctx
    rows = x_rows.shape[0]
    H, qd, F = cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.ffn
    d = {n: nat.buf(a) for n, a in w.items()}
    dx, dq, datt, dx1, dx1n = nat.buf(x_rows), nat.buf(rows * qd * 4), nat.buf(rows * qd * 4), nat.buf(rows * H * 4), nat.buf(rows * H * 4)
    dhid, dout = nat.buf(rows * F * 4), nat.buf(rows * H * 4)
    dids, dpos = nat.buf(np.asarray(seq_ids, np.uint32)), nat.buf(np.asarray(positions, np.uint32))
    dlens = nat.buf(np.asarray(positions, np.uint32) + 1)
    g = lambda n: d[n].ptr if n in d else None
    if one_call_front:  # steps 1-6 through the single entry point (one row: projection + one cluster kernel)
        rc = L.m40llm_qkv_rope_append_attention_async(ctx, kv, dx.ptr, d["attn_norm"].ptr, 1, cfg.eps, d["wq"].ptr,
                                                      d["wk"].ptr, d["wv"].ptr, g("bq"), g("bk"), g("bv"), dids.ptr, dpos.ptr,
                                                      dlens.ptr, rows, H, cfg.q_heads, cfg.rope_base, cfg.rope_scale,
                                                      cfg.rope_layout, dq.ptr, datt.ptr)
        assert rc == 0, rc
    else:
        rc = L.m40llm_qkv_rmsnorm_rope_append_async(ctx, kv, dx.ptr, d["attn_norm"].ptr, 1, cfg.eps, d["wq"].ptr, d["wk"].ptr,
                                                    d["wv"].ptr, g("bq"), g("bk"), g("bv"), dids.ptr, dpos.ptr, rows, H,
                                                    cfg.q_heads, cfg.rope_base, cfg.rope_scale, cfg.rope_layout, dq.ptr)
        assert rc == 0, rc
        assert L.m40llm_attention_last_token_f32_gqa_batched_async(ctx, kv, dids.ptr, dlens.ptr, rows, dq.ptr, cfg.q_heads, datt.ptr) == 0
    if fused_tail:
        rc = L.m40llm_attn_out_ffn_async(ctx, datt.ptr, d["wo"].ptr, dx.ptr, d["ffn_norm"].ptr, 1, cfg.eps, d["wg"].ptr,
                                         d["wu"].ptr, d["wd"].ptr, 1 if q80 else 0, dx1.ptr, dhid.ptr, dout.ptr, rows,
                                         H, qd, F)
        assert rc == 0, rc
        nat.sync(1)
        return (dout.download(np.float32, (rows, H)), dq.download(np.float32, (rows, qd)), datt.download(np.float32, (rows, qd)))
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
@pytest.mark.parametrize("fused_tail,one_call_front", [(False, False), (True, False), (True, True)])
def test_decode_layer_single_row(nat, O, H, qh, kvh, hd, F, q80, layout, bias, base, ctx_len, fused_tail, one_call_front):
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
        out, q_rot, att = device_layer(nat, kv, w, x[None, :], [0], [pos], cfg, q80, fused_tail, one_call_front)
        eout, eq, eatt = O.decode_layer(cfg, x, w, K, V, pos)
        k_dev, v_dev = np.zeros((kvh, hd), np.float16), np.zeros((kvh, hd), np.float16)
        assert nat.lib.m40llm_kvcache_debug_read_token(nat.ctx, kv, 0, pos, k_dev.ctypes.data_as(C.c_void_p),
                                                       v_dev.ctypes.data_as(C.c_void_p)) == 0
        assert_close(k_dev.astype(np.float32), K[pos].astype(np.float32), what=f"appended k, step {step}")
        assert_close(v_dev.astype(np.float32), V[pos].astype(np.float32), what=f"appended v, step {step}")
        assert_close(q_rot[0], eq, what=f"q after rope, step {step}")
        assert_close(att[0], eatt, what=f"attention, step {step}")
        assert_close(out[0], eout, what=f"layer output, step {step}")
        x = eout
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("fused_tail", [False, True])
def test_decode_layer_batched_rows_and_compressed_append(nat, O, fused_tail):
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
    out, q_rot, att = device_layer(nat, kv, w, x, list(range(B)), [n - 1 for n in lens], cfg, True, fused_tail)
    for b, n in enumerate(lens):
        eout, eq, eatt = O.decode_layer(cfg, x[b], w, Ks[b], Vs[b], n - 1)
        assert_close(q_rot[b], eq, what=f"row {b} q after rope")
        assert_close(att[b], eatt, what=f"row {b} attention")
        assert_close(out[b], eout, what=f"row {b} output")
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_batched_prologue_epilogue_rope_append_bias_and_bad_position(nat, O):
    """Batched rows on a dense cache with adjacent RoPE: the QKV projection's epilogue rotates q / k and appends k / v
    itself (no separate launch). With QKV bias; a row whose position lies outside the cache raises status bit 2 and
    leaves the cache alone while the other rows are appended (kernels.cu:1297-1346 checks the same bounds)."""
    rng = np.random.default_rng(123)
    H, qh, kvh, hd, F = 512, 8, 2, 64, 768
    cfg = O.LayerCfg(H, qh, kvh, hd, F, 0, 0, 1e-5, 5e5, 1.0)
    w = make_weights(O, rng, H, qh, kvh, hd, F, False, True)
    L, ctx = nat.lib, nat.ctx
    B, max_seq = 4, 96
    kv = nat.kv_dense(max_seq, B, kvh, hd)
    positions = [10, 95, 400, 0]  # row 2 is out of range
    x = rng.standard_normal((B, H)).astype(np.float32)
    d = {n: nat.buf(a) for n, a in w.items()}
    dx, dq = nat.buf(x), nat.buf(B * qh * hd * 4)
    dids, dpos = nat.buf(np.arange(B, dtype=np.uint32)), nat.buf(np.asarray(positions, np.uint32))
    rc = L.m40llm_qkv_rmsnorm_rope_append_async(ctx, kv, dx.ptr, d["attn_norm"].ptr, 1, cfg.eps, d["wq"].ptr, d["wk"].ptr,
                                                d["wv"].ptr, d["bq"].ptr, d["bk"].ptr, d["bv"].ptr, dids.ptr, dpos.ptr, B,
                                                H, qh, cfg.rope_base, cfg.rope_scale, 0, dq.ptr)
    assert rc == 0, rc
    nat.sync(1)
    st = np.zeros(1, np.uint32)
    assert L.m40llm_context_take_device_status(ctx, st.ctypes.data) == 0 and st[0] == 2
    q = dq.download(np.float32, (B, qh * hd))
    for b, pos in enumerate(positions):
        if pos >= max_seq:
            continue
        xn = O.rms_norm(x[b], w["attn_norm"], cfg.eps)
        eq = O.rope(O.gemm_f32xf16_gguf(xn, w["wq"]) + w["bq"], qh, hd, pos, cfg.rope_base, 1.0, 0)
        ek = O.rope(O.gemm_f32xf16_gguf(xn, w["wk"]) + w["bk"], kvh, hd, pos, cfg.rope_base, 1.0, 0)
        ev = O.gemm_f32xf16_gguf(xn, w["wv"]) + w["bv"]
        assert_close(q[b], eq, what=f"row {b} q")
        k_dev, v_dev = np.zeros((kvh, hd), np.float16), np.zeros((kvh, hd), np.float16)
        assert L.m40llm_kvcache_debug_read_token(ctx, kv, b, pos, k_dev.ctypes.data_as(C.c_void_p),
                                                 v_dev.ctypes.data_as(C.c_void_p)) == 0
        assert_close(k_dev.astype(np.float32).ravel(), O.f32_to_f16(ek).astype(np.float32).ravel(), what=f"row {b} k")
        assert_close(v_dev.astype(np.float32).ravel(), O.f32_to_f16(ev).astype(np.float32).ravel(), what=f"row {b} v")
    L.m40llm_kvcache_destroy(kv)
    nat.free_all()


def _host_weights(pkg, nat, w, q80):
    d = {n: nat.buf(a) for n, a in w.items()}
    W = pkg.host.Weights()
    for n in ("attn_norm", "ffn_norm", "wq", "wk", "wv", "wo", "bq", "bk", "bv", "wg", "wu", "wd"):
        setattr(W, n, d[n].ptr if n in d else None)
    W.ffn_q80 = 1 if q80 else 0
    return W


def test_host_layer_driver_dense_with_graph_replay(nat, O, pkg):
    """The C++ host mirror (forward_one_token...batched, src/infer/forward.rs:1729-2140) with HOST buffers: three
    consecutive steps of a 4-request batch (one request inactive); steps 2-3 replay the captured graph."""
    rng = np.random.default_rng(5)
    H, qh, kvh, hd, F = 512, 8, 2, 64, 1024
    cfg = O.LayerCfg(H, qh, kvh, hd, F, 1, 0, 1e-5, 1e4, 1.0)
    w = make_weights(O, rng, H, qh, kvh, hd, F, True, False)
    W = _host_weights(pkg, nat, w, True)
    lens = [40, 7, 130, 65]
    max_seq = 160
    kv = nat.kv_dense(max_seq, 4, kvh, hd)
    Ks = [np.zeros((max_seq, kvh, hd), np.float16) for _ in lens]
    Vs = [np.zeros((max_seq, kvh, hd), np.float16) for _ in lens]
    for b, n in enumerate(lens):
        Ks[b][:n] = rng.standard_normal((n, kvh, hd)).astype(np.float16)
        Vs[b][:n] = rng.standard_normal((n, kvh, hd)).astype(np.float16)
        nat.kv_fill(kv, b, Ks[b][:n], Vs[b][:n])
    layer = pkg.host.DecodeLayer(nat.ctx, pkg.host.LayerCfg(H, qh, kvh, hd, F, 0, 1e-5, 1e4, 1.0), 8)
    active = [0, 2, 3]
    x = rng.standard_normal((3, H)).astype(np.float32)
    for step in range(3):
        reqs = [(100 + b, b, lens[b] + step + 1, b in active) for b in range(4)]
        out = layer.forward_host(kv, W, pkg.host.dense_kv_cfg(), reqs, x, use_graph=True)
        for i, b in enumerate(active):
            eout, _, _ = O.decode_layer(cfg, x[i], w, Ks[b], Vs[b], lens[b] + step)
            assert_close(out[i], eout, what=f"step {step} request {b}")
        x = out.copy()
    assert layer.graph_replays() >= 1
    with pytest.raises(RuntimeError, match="at least one active request"):
        layer.forward_host(kv, W, pkg.host.dense_kv_cfg(), [(1, 0, 5, False)], x[:1])
    layer.close()
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_host_layer_driver_two_steps_in_flight(nat, O, pkg):
    """forward_host in its two halves: two micro-batches (sequences 0-1 and 2-3 of one cache) ping-pong through the
    two slots, each begun before the other is ended; three steps each, checked against the oracle layer."""
    rng = np.random.default_rng(15)
    H, qh, kvh, hd, F = 512, 8, 2, 64, 1024
    cfg = O.LayerCfg(H, qh, kvh, hd, F, 1, 0, 1e-5, 1e4, 1.0)
    w = make_weights(O, rng, H, qh, kvh, hd, F, True, False)
    W = _host_weights(pkg, nat, w, True)
    lens = [33, 90, 12, 140]
    max_seq = 160
    kv = nat.kv_dense(max_seq, 4, kvh, hd)
    Ks = [np.zeros((max_seq, kvh, hd), np.float16) for _ in lens]
    Vs = [np.zeros((max_seq, kvh, hd), np.float16) for _ in lens]
    for b, n in enumerate(lens):
        Ks[b][:n] = rng.standard_normal((n, kvh, hd)).astype(np.float16)
        Vs[b][:n] = rng.standard_normal((n, kvh, hd)).astype(np.float16)
        nat.kv_fill(kv, b, Ks[b][:n], Vs[b][:n])
    layer = pkg.host.DecodeLayer(nat.ctx, pkg.host.LayerCfg(H, qh, kvh, hd, F, 0, 1e-5, 1e4, 1.0), 8)
    kc = pkg.host.dense_kv_cfg()
    groups = [[0, 1], [2, 3]]
    xs = [np.ascontiguousarray(rng.standard_normal((2, H)).astype(np.float32)) for _ in groups]
    outs = [np.zeros((2, H), np.float32) for _ in groups]
    p = lambda a: a.ctypes.data_as(C.c_void_p)

    def begin(slot, step):
        seqs = groups[slot]
        rid = np.array([100 + b for b in seqs], np.uint64)
        sid = np.array(seqs, np.uint32)
        kvl = np.array([lens[b] + step + 1 for b in seqs], np.uint32)
        act = np.ones(2, np.uint32)
        return layer.forward_host_begin_raw(slot, kv, W, kc, 2, p(rid), p(sid), p(kvl), p(act), p(xs[slot]), True)

    assert begin(0, 0) == 0
    # a busy slot cannot be begun again, and an idle one cannot be ended
    assert begin(0, 0) != 0
    assert layer.forward_host_end_raw(1, p(outs[1])) != 0
    for step in range(3):
        assert begin(1, step) == 0
        for slot in (0, 1):
            assert layer.forward_host_end_raw(slot, p(outs[slot])) == 0
            for i, b in enumerate(groups[slot]):
                eout, _, _ = O.decode_layer(cfg, xs[slot][i], w, Ks[b], Vs[b], lens[b] + step)
                assert_close(outs[slot][i], eout, what=f"step {step} slot {slot} sequence {b}")
            xs[slot][:] = outs[slot]
            if slot == 0 and step + 1 < 3:
                assert begin(0, step + 1) == 0
    layer.close()
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_host_layer_driver_compressed_mode(nat, O, pkg):
    """Attention-mode dispatch (src/infer/kv.rs:433-765): BlockSelectExact + FP16-K/q4-V direct on a compressed cache,
    Qwen-style heads (NeoX RoPE, QKV bias). The layer appends through the ring (with eviction) and attends."""
    rng = np.random.default_rng(6)
    H, qh, kvh, hd, F = 256, 8, 2, 128, 512
    R, bs, top, L0 = 16, 8, 3, 90
    w = make_weights(O, rng, H, qh, kvh, hd, F, False, True)
    W = _host_weights(pkg, nat, w, False)
    kv = nat.kv_compressed(128, 1, kvh, hd, R, bs, top)
    k16 = rng.standard_normal((L0, kvh, hd)).astype(np.float16)
    v16 = rng.standard_normal((L0, kvh, hd)).astype(np.float16)
    nat.kv_fill(kv, 0, k16, v16, final_len=L0)
    kc = pkg.host.default_kv_cfg()
    kc.recent_window, kc.block_size, kc.top_blocks = R, bs, top
    layer = pkg.host.DecodeLayer(nat.ctx, pkg.host.LayerCfg(H, qh, kvh, hd, F, 1, 1e-5, 1e6, 1.0), 2)
    x = rng.standard_normal((1, H)).astype(np.float32)
    out = layer.forward_host(kv, W, kc, [(7, 0, L0 + 1, True)], x)
    # oracle: the same ops composed by hand around the compressed attention
    xn = O.rms_norm(x[0], w["attn_norm"], 1e-5)
    q = O.rope(O.gemm_f32xf16_gguf(xn, w["wq"]) + w["bq"], qh, hd, L0, 1e6, 1.0, 1)
    k = O.rope(O.gemm_f32xf16_gguf(xn, w["wk"]) + w["bk"], kvh, hd, L0, 1e6, 1.0, 1)
    v = O.gemm_f32xf16_gguf(xn, w["wv"]) + w["bv"]
    kall = np.concatenate([k16, O.f32_to_f16(k).reshape(1, kvh, hd)])
    vall = np.concatenate([v16, O.f32_to_f16(v).reshape(1, kvh, hd)])
    old_k, q4, sc, rk, rv = O.compressed_state_from_dense(kall, vall, L0 + 1, R)
    att, *_ = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, L0 + 1, R, bs, top)
    x1 = x[0] + O.gemm_f32xf16_gguf(att, w["wo"])
    x1n = O.rms_norm(x1, w["ffn_norm"], 1e-5)
    hid = O.swiglu(O.gemm_f32xf16_gguf(x1n, w["wg"]), O.gemm_f32xf16_gguf(x1n, w["wu"]))
    assert_close(out[0], x1 + O.gemm_f32xf16_gguf(hid, w["wd"]), what="compressed-mode layer")
    bad = pkg.host.default_kv_cfg()
    bad.exact_old_backing, bad.exact_old_attention = 1, 1
    with pytest.raises(RuntimeError, match="head_dim=128"):  # the reference refuses q8 backing at head_dim 128 too
        layer.forward_host(kv, W, bad, [(7, 0, L0 + 2, True)], x)
    layer.close()
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_graph_replay_survives_scratch_growth(O, pkg):
    """A captured layer graph has the scratch arena's addresses baked in. A later eager call that needs a larger
    arena must not invalidate it: small batch with graph -> a call that outgrows the arena -> the small batch's graph
    again, every step against the oracle. Runs on a context of its own so that the arena starts at its initial size."""
    import helpers

    own = helpers.Native(pkg.native.lib())
    try:
        rng = np.random.default_rng(15)
        H, qh, kvh, hd, F = 512, 8, 2, 64, 1024
        cfg = O.LayerCfg(H, qh, kvh, hd, F, 1, 0, 1e-5, 1e4, 1.0)
        w = make_weights(O, rng, H, qh, kvh, hd, F, True, False)
        W = _host_weights(pkg, own, w, True)
        lens = [300, 7, 130, 65]
        max_seq = 320
        kv = own.kv_dense(max_seq, 4, kvh, hd)
        Ks = [np.zeros((max_seq, kvh, hd), np.float16) for _ in lens]
        Vs = [np.zeros((max_seq, kvh, hd), np.float16) for _ in lens]
        for b, n in enumerate(lens):
            Ks[b][:n] = rng.standard_normal((n, kvh, hd)).astype(np.float16)
            Vs[b][:n] = rng.standard_normal((n, kvh, hd)).astype(np.float16)
            own.kv_fill(kv, b, Ks[b][:n], Vs[b][:n])
        layer = pkg.host.DecodeLayer(own.ctx, pkg.host.LayerCfg(H, qh, kvh, hd, F, 0, 1e-5, 1e4, 1.0), 4)
        x = rng.standard_normal((4, H)).astype(np.float32)

        def generation():
            g = np.zeros(1, np.uint64)
            assert own.lib.m40llm_context_scratch_generation(own.ctx, g.ctypes.data) == 0
            return int(g[0])

        def step(i):
            nonlocal x
            reqs = [(b, b, lens[b] + i + 1, True) for b in range(4)]
            out = layer.forward_host(kv, W, pkg.host.dense_kv_cfg(), reqs, x, use_graph=True)
            for b in range(4):
                eout, _, _ = O.decode_layer(cfg, x[b], w, Ks[b], Vs[b], lens[b] + i)
                assert_close(out[b], eout, what=f"step {i} row {b}")
            x = out.copy()

        step(0)  # eager + capture
        step(1)  # replay
        assert layer.graph_replays() == 1
        g0 = generation()
        # 256 rows x 64 q heads x 8 splits x (2 + 64) floats of attention partials = 34.6 MB > the 32 MB arena
        big_rows, bq, bkv, bhd, bmax = 256, 64, 4, 64, 8192
        big = own.kv_dense(bmax, big_rows, bkv, bhd)
        dq = own.buf(rng.standard_normal((big_rows, bq * bhd)).astype(np.float32))
        do = own.buf(big_rows * bq * bhd * 4)
        dids = own.buf(np.arange(big_rows, dtype=np.uint32))
        dlens = own.buf(np.full(big_rows, bmax, np.uint32))
        assert own.lib.m40llm_attention_last_token_f32_gqa_batched_async(own.ctx, big, dids.ptr, dlens.ptr, big_rows,
                                                                         dq.ptr, bq, do.ptr) == 0
        own.sync(1)
        assert generation() > g0, "the large call was meant to outgrow the scratch arena"
        step(2)  # replays the graph captured against the old arena
        step(3)
        assert layer.graph_replays() == 3
        layer.close()
        own.lib.m40llm_kvcache_destroy(big)
        own.lib.m40llm_kvcache_destroy(kv)
    finally:
        own.free_all()
        own.lib.m40llm_destroy_context(own.ctx)


def _batched_layer_case(nat, O, H, qh, kvh, hd, F, base, lens, fused_tail, seed, check_rows=None):
    """Fills a dense cache with `lens[b] - 1` random tokens per sequence, runs the batched layer for one new token per
    sequence and compares rows (all, or `check_rows`) with the oracle's single-sequence layer, including the K/V row
    the prologue appended."""
    rng = np.random.default_rng(seed)
    cfg = O.LayerCfg(H, qh, kvh, hd, F, 1, 0, 1e-5, base, 1.0)
    w = make_weights(O, rng, H, qh, kvh, hd, F, True, False)
    B, max_seq = len(lens), max(lens) + 2
    kv = nat.kv_dense(max_seq, B, kvh, hd)
    pre = {}
    for b, n in enumerate(lens):
        k = rng.standard_normal((n - 1, kvh, hd), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((n - 1, kvh, hd), dtype=np.float32).astype(np.float16)
        if n > 1:
            nat.kv_fill(kv, b, k, v)
        pre[b] = (k, v)
    x = rng.standard_normal((B, H)).astype(np.float32)
    out, q_rot, att = device_layer(nat, kv, w, x, list(range(B)), [n - 1 for n in lens], cfg, True, fused_tail)
    for b in (range(B) if check_rows is None else check_rows):
        n = lens[b]
        K = np.zeros((n + 1, kvh, hd), np.float16)
        V = np.zeros((n + 1, kvh, hd), np.float16)
        K[:n - 1], V[:n - 1] = pre[b]
        eout, eq, eatt = O.decode_layer(cfg, x[b], w, K, V, n - 1)
        assert_close(q_rot[b], eq, what=f"row {b} q after rope")
        assert_close(att[b], eatt, what=f"row {b} attention")
        assert_close(out[b], eout, what=f"row {b} output")
        k_dev, v_dev = np.zeros((kvh, hd), np.float16), np.zeros((kvh, hd), np.float16)
        assert nat.lib.m40llm_kvcache_debug_read_token(nat.ctx, kv, b, n - 1, k_dev.ctypes.data_as(C.c_void_p),
                                                       v_dev.ctypes.data_as(C.c_void_p)) == 0
        assert_close(k_dev.astype(np.float32), K[n - 1].astype(np.float32), what=f"row {b} appended k")
        assert_close(v_dev.astype(np.float32), V[n - 1].astype(np.float32), what=f"row {b} appended v")
    st = np.zeros(1, np.uint32)
    assert nat.lib.m40llm_context_take_device_status(nat.ctx, st.ctypes.data) == 0 and st[0] == 0
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("fused_tail", [False, True])
def test_llama3_8b_layer_32_rows(nat, O, fused_tail):
    """The configuration the benchmark is quoted on, as a whole: hidden 4096, 32/8 heads of 128, Q8_0 FFN 14336,
    RoPE theta 5e5 applied by the projection's epilogue, 32 rows with contexts between 512 and 8192."""
    lens = [int(n) for n in np.random.default_rng(0).integers(512, 8193, size=32)]
    lens[3], lens[17] = 512, 8192
    _batched_layer_case(nat, O, 4096, 32, 8, 128, 14336, 5e5, lens, fused_tail, seed=4096 + 32)


@pytest.mark.parametrize("rows,H,qh,kvh,hd,F", [(65, 512, 8, 2, 64, 1024),      # a trailing single row after a 64-row pass
                                                 (128, 1024, 8, 2, 128, 2816),   # two passes, head_dim 128 epilogue
                                                 (256, 512, 4, 1, 128, 768)])    # four passes
def test_batched_layer_many_rows(nat, O, rows, H, qh, kvh, hd, F):
    """Row counts of the batch sweep (128, 256) and the 64k+1 case, where the FFN norm cannot ride on the tensor-core
    path's activation split; every 7th row and the last are compared."""
    lens = [int(n) for n in np.random.default_rng(rows).integers(1, 300, size=rows)]
    rows_to_check = sorted(set(range(0, rows, 7)) | {rows - 1, 63, 64})
    _batched_layer_case(nat, O, H, qh, kvh, hd, F, 5e5, lens, True, seed=rows, check_rows=rows_to_check)


@pytest.mark.parametrize("qh,kvh,hd,layout,ctx_len", [
    (8, 2, 64, 0, 0),        # empty cache: the new token is the only one attended
    (8, 2, 64, 1, 1),
    (32, 8, 128, 0, 63), (32, 8, 128, 0, 64), (32, 8, 128, 0, 65),   # around one tile
    (32, 8, 128, 0, 1023), (32, 8, 128, 0, 1024), (32, 8, 128, 0, 1025),  # around 16 slices of one tile
    (16, 2, 128, 1, 5000),   # Qwen heads, NeoX RoPE
    (32, 4, 64, 0, 2048),    # TinyLlama heads
    (32, 2, 64, 0, 777),     # 16 q heads per kv head (rows 8..15 of the MMA live)
    (24, 8, 128, 0, 300),    # 3 q heads per kv head
    (32, 8, 128, 0, 16383),
])
def test_one_launch_row_attention(nat, O, qh, kvh, hd, layout, ctx_len):
    """m40llm_qkv_rope_append_attention_async at one row against the op-by-op oracle: q after RoPE, the appended K/V
    row, the recorded sequence length and the attention output, at contexts around the kernel's slice boundaries."""
    rng = np.random.default_rng(ctx_len + qh + hd)
    H, base = 256, 5e5
    w = make_weights(O, rng, H, qh, kvh, hd, 128, False, True)
    max_seq = ctx_len + 3
    K = np.zeros((max_seq, kvh, hd), np.float16)
    V = np.zeros((max_seq, kvh, hd), np.float16)
    K[:ctx_len] = rng.standard_normal((ctx_len, kvh, hd)).astype(np.float16)
    V[:ctx_len] = rng.standard_normal((ctx_len, kvh, hd)).astype(np.float16)
    kv = nat.kv_dense(max_seq, 2, kvh, hd)
    if ctx_len:
        nat.kv_fill(kv, 1, K[:ctx_len], V[:ctx_len])
    L, ctx = nat.lib, nat.ctx
    d = {n: nat.buf(a) for n, a in w.items()}
    x = rng.standard_normal((1, H)).astype(np.float32)
    dx, dq, datt = nat.buf(x), nat.buf(qh * hd * 4), nat.buf(qh * hd * 4)
    dids, dpos, dlens = nat.buf(np.array([1], np.uint32)), nat.buf(np.array([ctx_len], np.uint32)), nat.buf(np.array([ctx_len + 1], np.uint32))
    call = lambda: L.m40llm_qkv_rope_append_attention_async(
        ctx, kv, dx.ptr, d["attn_norm"].ptr, 1, 1e-5, d["wq"].ptr, d["wk"].ptr, d["wv"].ptr, d["bq"].ptr, d["bk"].ptr,
        d["bv"].ptr, dids.ptr, dpos.ptr, dlens.ptr, 1, H, qh, base, 1.0, layout, dq.ptr, datt.ptr)
    assert call() == 0
    nat.sync(1)
    xn = O.rms_norm(x[0], w["attn_norm"], 1e-5)
    eq = O.rope(O.gemm_f32xf16_gguf(xn, w["wq"]) + w["bq"], qh, hd, ctx_len, base, 1.0, layout)
    ek = O.f32_to_f16(O.rope(O.gemm_f32xf16_gguf(xn, w["wk"]) + w["bk"], kvh, hd, ctx_len, base, 1.0, layout)).reshape(kvh, hd)
    ev = O.f32_to_f16(O.gemm_f32xf16_gguf(xn, w["wv"]) + w["bv"]).reshape(kvh, hd)
    K[ctx_len], V[ctx_len] = ek, ev
    assert_close(dq.download(np.float32, (qh * hd,)), eq, what="q after rope")
    k_dev, v_dev = np.zeros((kvh, hd), np.float16), np.zeros((kvh, hd), np.float16)
    assert L.m40llm_kvcache_debug_read_token(ctx, kv, 1, ctx_len, k_dev.ctypes.data_as(C.c_void_p), v_dev.ctypes.data_as(C.c_void_p)) == 0
    assert_close(k_dev.astype(np.float32), ek.astype(np.float32), what="appended k")
    assert_close(v_dev.astype(np.float32), ev.astype(np.float32), what="appended v")
    assert_close(datt.download(np.float32, (qh * hd,)), O.attention_gqa(K, V, eq, qh, ctx_len + 1), what="attention")
    st = np.zeros(1, np.uint32)
    assert L.m40llm_context_take_device_status(ctx, st.ctypes.data) == 0 and st[0] == 0
    # the one-launch path needs the new token to be the last attended one: otherwise the row is flagged and zeroed
    dlens.upload(np.array([ctx_len + 2], np.uint32))
    datt.upload(np.full(qh * hd, 3.0, np.float32))
    assert call() == 0
    assert L.m40llm_context_take_device_status(ctx, st.ctypes.data) == 0 and st[0] == 1
    assert not datt.download(np.float32, (qh * hd,)).any()
    L.m40llm_kvcache_destroy(kv)
    nat.free_all()
