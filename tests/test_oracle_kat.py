"""The oracle against independent numpy (float64) restatements, on the closed-form inputs the
reference's own tests use. Each case names the reference test it mirrors.

These run on CPU. They pin the oracle's arithmetic; the golden fixtures made by the reference's
own CUDA code (test_oracle_golden.py) pin it against the reference itself.
"""
import numpy as np
import pytest


def np_attention(q, k, v, q_heads):
    """float64 softmax attention; k, v [L, Hkv, hd] (already f16-rounded values)."""
    L, hkv, hd = k.shape
    g = q_heads // hkv
    out = np.zeros((q_heads, hd))
    for h in range(q_heads):
        s = k[:, h // g, :].astype(np.float64) @ q[h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        p /= p.sum()
        out[h] = p @ v[:, h // g, :].astype(np.float64)
    return out.ravel()


def closed_form_kv(seq_len, dim):
    """tests/attention_parity_cpu_grid.rs:91-119: k = (t*dim+i)*0.01-1, v = (t*dim+(dim-1-i))*0.02-2, q = i*0.003-0.5."""
    t = np.arange(seq_len, dtype=np.float32)[:, None]
    i = np.arange(dim, dtype=np.float32)[None, :]
    k = (t * dim + i) * np.float32(0.01) - np.float32(1.0)
    v = (t * dim + (dim - 1 - i)) * np.float32(0.02) - np.float32(2.0)
    q = np.arange(dim, dtype=np.float32) * np.float32(0.003) - np.float32(0.5)
    return k.astype(np.float32), v.astype(np.float32), q


def test_f16_round_trip_matches_ieee(O):
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-2, 1.0, 300.0, 6e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, 65504.0, 65519.0, 65520.0, 5.96e-8, 2.98e-8, 2.9802322e-8, 1e-10],
                                    dtype=np.float32)])
    with np.errstate(over="ignore"):
        expect = x.astype(np.float16)
    assert np.array_equal(O.f32_to_f16(x).view(np.uint16), expect.view(np.uint16))
    allh = np.arange(65536, dtype=np.uint16).view(np.float16)
    got = O.f16_to_f32(allh)
    ref = allh.astype(np.float32)
    ok = (got.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(got) & np.isnan(ref))
    assert ok.all()


@pytest.mark.parametrize("heads", [1, 2, 3, 4])
@pytest.mark.parametrize("hd", [1, 5, 7, 8, 16, 31, 32, 63, 64])
def test_mha_cpu_grid(O, heads, hd):
    """tests/attention_parity_cpu_grid.rs:74-119 (tolerance 1e-6 there; float64 reference here)."""
    dim = heads * hd
    for seq_len in (1, 2, 3, 4, 7, 8, 16):
        k, v, q = closed_form_kv(seq_len, dim)
        k16 = O.f32_to_f16(k).reshape(seq_len, heads, hd)
        v16 = O.f32_to_f16(v).reshape(seq_len, heads, hd)
        got = O.attention_gqa(k16, v16, q, heads, seq_len)
        ref = np_attention(q, k16, v16, heads)
        np.testing.assert_allclose(got, ref, atol=2e-6, rtol=2e-6)


@pytest.mark.parametrize("qh,kvh", [(2, 1), (4, 1), (8, 2), (32, 4)])
@pytest.mark.parametrize("hd", [1, 5, 8, 16, 32, 128])
def test_gqa_grid(O, qh, kvh, hd):
    """tests/attention_parity_cuda_grid.rs:1625-1667 head pairs and head dims."""
    rng = np.random.default_rng(qh * 1000 + hd)
    for seq_len in (1, 3, 17, 64):
        k = rng.standard_normal((seq_len, kvh, hd)).astype(np.float16)
        v = rng.standard_normal((seq_len, kvh, hd)).astype(np.float16)
        q = rng.standard_normal(qh * hd).astype(np.float32)
        got = O.attention_gqa(k, v, q, qh, seq_len)
        np.testing.assert_allclose(got, np_attention(q, k, v, qh), atol=5e-6, rtol=1e-5)


def test_batched_equals_per_sequence(O):
    """tests/attention_batched_varlen.rs:36-71: q4/kv2/hd64, lens {1,3,5}."""
    rng = np.random.default_rng(7)
    slots, max_seq, kvh, hd, qh = 4, 8, 2, 64, 4
    k = rng.standard_normal((slots, max_seq, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((slots, max_seq, kvh, hd)).astype(np.float16)
    ids = np.array([2, 0, 3], dtype=np.uint32)
    lens = np.array([1, 3, 5], dtype=np.uint32)
    q = rng.standard_normal((3, qh, hd)).astype(np.float32)
    out = O.attention_gqa_batched(k, v, ids, lens, q, qh)
    for b in range(3):
        one = O.attention_gqa(k[ids[b]], v[ids[b]], q[b].ravel(), qh, int(lens[b]))
        assert np.array_equal(out[b].ravel(), one)


def test_rms_norm_kat(O):
    """tests/rmsnorm_rope.rs:85-89, 127-132."""
    x = (np.arange(16, dtype=np.float32) * np.float32(0.25) - np.float32(3.0)).reshape(2, 8)
    got = O.rms_norm(x, None, 1e-5)
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
    np.testing.assert_allclose(got, ref, atol=1e-6)
    x = (np.arange(16, dtype=np.float32) * np.float32(0.125) - np.float32(1.0)).reshape(2, 8)
    w = (0.5 + np.arange(8, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    got = O.rms_norm(x, w, 1e-5)
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5) * w
    np.testing.assert_allclose(got, ref, atol=1e-6)


@pytest.mark.parametrize("layout", [0, 1])
def test_rope_kat(O, layout):
    """tests/rmsnorm_rope.rs:242-252 (adjacent); NeoX pairing per cuda/kernels.cu:5570-5585."""
    heads, hd, past = 2, 4, 3
    x = np.arange(heads * hd, dtype=np.float32) * np.float32(0.1) + np.float32(0.5)
    got = O.rope(x, heads, hd, past, 10000.0, 1.0, layout).reshape(heads, hd)
    xr = x.reshape(heads, hd).astype(np.float64)
    ref = xr.copy()
    for i in range(hd // 2):
        th = past * 10000.0 ** (-2.0 * i / hd)
        i0, i1 = (i, i + hd // 2) if layout == 1 else (2 * i, 2 * i + 1)
        ref[:, i0] = xr[:, i0] * np.cos(th) - xr[:, i1] * np.sin(th)
        ref[:, i1] = xr[:, i0] * np.sin(th) + xr[:, i1] * np.cos(th)
    np.testing.assert_allclose(got, ref, atol=1e-5)
    # larger: positions where f32 trig matters; layouts must only differ by the pairing permutation
    rng = np.random.default_rng(3)
    heads, hd = 3, 128
    x = rng.standard_normal(heads * hd).astype(np.float32)
    a = O.rope(x, heads, hd, 4097, 500000.0, 1.0, 0).reshape(heads, hd)
    xn = x.reshape(heads, hd)
    perm = np.concatenate([np.arange(0, hd, 2), np.arange(1, hd, 2)])  # adjacent -> neox element order
    b = O.rope(xn[:, perm].ravel(), heads, hd, 4097, 500000.0, 1.0, 1).reshape(heads, hd)
    assert np.array_equal(a[:, perm], b)


def test_gemm_forms(O):
    """tests/gemm_f16xf16_f32.rs:26-38, tests/gemm_mixed.rs:63-102, tests/forward_parity_toy.rs:30-43."""
    rng = np.random.default_rng(5)
    M, N, K = 3, 10, 37
    a = rng.standard_normal((M, K)).astype(np.float32)
    a16 = a.astype(np.float16)
    b16 = rng.standard_normal((K, N)).astype(np.float16)
    np.testing.assert_allclose(O.gemm_f16xf16_rowmajor(a16, b16), a16.astype(np.float64) @ b16.astype(np.float64), atol=1e-4)
    np.testing.assert_allclose(O.gemm_f32xf16_rowmajor(a, b16), a.astype(np.float64) @ b16.astype(np.float64), atol=1e-4)
    w = np.ascontiguousarray(b16.T)  # GGUF layout [N][K]
    np.testing.assert_allclose(O.gemm_f32xf16_gguf(a, w), a.astype(np.float64) @ b16.astype(np.float64), atol=1e-4)
    c16 = O.gemm_f16_storage(a16, b16)
    assert np.array_equal(c16.view(np.uint16), O.f32_to_f16(O.gemm_f16xf16_rowmajor(a16, b16)).view(np.uint16))


def test_q80_format(O):
    """src/infer/embeddings.rs:80-140: 34-byte blocks {f16 d; i8 q[32]}, value d*q."""
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((5, 96)) * 0.02).astype(np.float32)
    q = O.q80_quantize(w)
    assert q.shape == (5, 96 // 32 * 34)
    deq = O.q80_to_f32(q, w.size).reshape(w.shape)
    blocks = q.reshape(5, 3, 34)
    d = blocks[:, :, :2].copy().view(np.float16).astype(np.float32)[..., 0]
    qs = blocks[:, :, 2:].view(np.int8).astype(np.float32)
    assert np.array_equal(deq, (d[..., None] * qs).reshape(5, 96))
    assert np.abs(deq - w).max() <= np.abs(w).max() / 127 * 0.51 + 1e-6
    x = rng.standard_normal((2, 96)).astype(np.float32)
    np.testing.assert_allclose(O.gemm_f32xq80_gguf(x, q, 5), x.astype(np.float64) @ deq.astype(np.float64).T, atol=1e-5)


def test_swiglu(O):
    g = np.linspace(-6, 6, 25, dtype=np.float32)
    u = np.linspace(2, -1, 25, dtype=np.float32)
    ref = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u
    np.testing.assert_allclose(O.swiglu(g, u), ref, atol=1e-6)


def test_q4_quantiser_matches_reference_test_formula(O):
    """tests/attention_parity_cuda_grid.rs:1471-1505 restated in numpy. The test there rounds half away
    from zero and clamps to [-8, 7]; the kernel (cuda/kernels.cu:2254-2258) rounds half to even and clamps
    to [-7, 7]. With scale = max/7 no value exceeds 7 in magnitude, so the two agree except at exact .5 ties."""
    rng = np.random.default_rng(11)
    v = rng.standard_normal((40, 2, 128)).astype(np.float16)
    packed, scale = O.q4_quantize(v)
    deq = O.q4_dequant(packed, scale)
    vf = v.astype(np.float32)
    mx = np.abs(vf).max(axis=-1)
    sc = np.where(mx > 0, mx / np.float32(7.0), np.float32(1.0 / 7.0)).astype(np.float32)
    assert np.array_equal(sc, scale)
    ratio = vf / sc[..., None]
    qref = np.clip(np.sign(ratio) * np.floor(np.abs(ratio) + 0.5), -8, 7)
    ties = np.isclose(np.abs(ratio) % 1.0, 0.5, atol=1e-6)
    ref = (qref * sc[..., None]).astype(np.float16).astype(np.float32)
    assert np.array_equal(deq[~ties], ref[~ties])
    zero = np.zeros((1, 1, 64), np.float16)
    p0, s0 = O.q4_quantize(zero)
    assert s0[0, 0] == np.float32(1.0 / 7.0) and not p0.any()


def np_block_select(old_k, qh, kvh, old_len, bs, top):
    nb = (old_len + bs - 1) // bs if old_len else 0
    k = old_k[:old_len, kvh, :].astype(np.float64)
    sc = np.array([(k[b * bs:min((b + 1) * bs, old_len)] @ qh.astype(np.float64)).sum() / (min((b + 1) * bs, old_len) - b * bs)
                   for b in range(nb)]) / np.sqrt(old_k.shape[2])
    order = sorted(range(nb), key=lambda b: (-sc[b], b))
    return order[:min(top, nb)], sc


def test_block_selection(O):
    """cuda/kernels.cu:2893-2930, 6526-6600: mean q.K score, top-k, ties to the lower index."""
    rng = np.random.default_rng(13)
    old_len, kvh, hd, bs, top = 1000, 2, 64, 32, 8
    old_k = rng.standard_normal((old_len, kvh, hd)).astype(np.float16)
    q = rng.standard_normal(hd).astype(np.float32)
    blocks, bscores, s32, s64 = O.block_select_head(old_k, q, 1, old_len, bs, top)
    ref_blocks, ref_sc = np_block_select(old_k, q, 1, old_len, bs, top)
    assert list(blocks) == ref_blocks
    np.testing.assert_allclose(s64, ref_sc, atol=1e-12)
    np.testing.assert_allclose(s32, ref_sc, atol=2e-6)
    assert np.all(np.diff(bscores) <= 0)
    # ties: identical blocks -> lowest indices win, in index order
    same = np.tile(old_k[:bs], (6, 1, 1))
    blocks, *_ = O.block_select_head(same, q, 0, 6 * bs, bs, 3)
    assert list(blocks) == [0, 1, 2]
    # NaN scores are never selected
    bad = old_k[:4 * bs].copy()
    bad[bs:2 * bs, 0, 0] = np.float16(np.nan)
    blocks, *_ = O.block_select_head(bad, q, 0, 4 * bs, bs, 4)
    assert 1 not in blocks and len(blocks) == 3


def test_compressed_attention_equals_dense_when_all_blocks_selected(O):
    """tests/attention_parity_cuda_grid.rs:216-306: q4/kv2/hd64, seq 16, R 4, bs 4, top 3 (all 3 old blocks)."""
    rng = np.random.default_rng(17)
    qh, kvh, hd, L, R, bs, top = 4, 2, 64, 16, 4, 4, 3
    k = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k, v, L, R)
    out, sel, cnt, union = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, L, R, bs, top)
    assert list(cnt) == [3] * qh and union == kvh * 12
    v_mixed = v.copy()
    v_mixed[:L - R] = O.q4_dequant(q4, sc).astype(np.float16)
    np.testing.assert_allclose(out, np_attention(q, k, v_mixed, qh), atol=5e-6, rtol=1e-5)
    dense = O.attention_block_select_dense(k, v, q, qh, L, R, bs, top)
    np.testing.assert_allclose(dense, np_attention(q, k, v, qh), atol=5e-6, rtol=1e-5)


def test_compressed_partial_block_and_short_sequences(O):
    """tests/attention_parity_cuda_grid.rs:618-673: hd128, seq 5, R 4, bs 32, top 8 (one partial block);
    and seq_len <= R (no old region at all)."""
    qh, kvh, hd = 4, 2, 128
    kv_dim = kvh * hd
    for L in (5, 4, 1):
        t = np.arange(L)[:, None]
        i = np.arange(kv_dim)[None, :]
        k = ((t * 17 + i * 3).astype(np.float32) * np.float32(0.0005) - np.float32(0.2)).astype(np.float32)
        v = ((t * 23 + kv_dim - i).astype(np.float32) * np.float32(0.0006) - np.float32(0.1)).astype(np.float32)
        q = np.arange(qh * hd, dtype=np.float32) * np.float32(0.0002) - np.float32(0.04)
        k16 = O.f32_to_f16(k).reshape(L, kvh, hd)
        v16 = O.f32_to_f16(v).reshape(L, kvh, hd)
        old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k16, v16, L, 4)
        out, sel, cnt, _ = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, L, 4, 32, 8)
        v_mixed = v16.copy()
        if L > 4:
            v_mixed[:L - 4] = O.q4_dequant(q4, sc).astype(np.float16)
        np.testing.assert_allclose(out, np_attention(q, k16, v_mixed, qh), atol=5e-6, rtol=1e-5)
        assert list(cnt) == [1 if L > 4 else 0] * qh


def test_compressed_selects_subset(O):
    rng = np.random.default_rng(19)
    qh, kvh, hd, L, R, bs, top = 8, 2, 128, 700, 64, 16, 5
    k = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k, v, L, R)
    out, sel, cnt, union = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, L, R, bs, top)
    vq = O.q4_dequant(q4, sc)
    for h in range(qh):
        ref_blocks, _ = np_block_select(old_k, q[h * hd:(h + 1) * hd], h // 4, L - R, bs, top)
        assert list(sel[h, :cnt[h]]) == ref_blocks
        toks = [t for b in ref_blocks for t in range(b * bs, min((b + 1) * bs, L - R))]
        kk = np.concatenate([old_k[toks, h // 4], k[L - R:, h // 4]]).astype(np.float64)
        vv = np.concatenate([vq[toks, h // 4], v[L - R:, h // 4].astype(np.float32)]).astype(np.float64)
        s = kk @ q[h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        p /= p.sum()
        np.testing.assert_allclose(out[h * hd:(h + 1) * hd], p @ vv, atol=5e-6, rtol=1e-5)
    assert top * bs * kvh <= union <= top * bs * qh


def test_merge_partials_identity(O):
    """Split-K: merging per-range partials reproduces attention over the whole range."""
    rng = np.random.default_rng(23)
    qh, kvh, hd, L = 8, 2, 64, 300
    k = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    bounds = [0, 90, 90, 211, 300]  # includes an empty part
    parts = len(bounds) - 1
    m = np.full((parts, qh), -np.inf, np.float32)
    l = np.zeros((parts, qh), np.float32)
    o = np.zeros((parts, qh, hd), np.float32)
    for r in range(parts):
        a, b = bounds[r], bounds[r + 1]
        if a == b:
            continue
        for h in range(qh):
            s = (k[a:b, h // 4].astype(np.float32) @ q[h * hd:(h + 1) * hd]) / np.float32(8.0)
            m[r, h] = s.max()
            e = np.exp(s - s.max())
            l[r, h] = e.sum()
            o[r, h] = e @ v[a:b, h // 4].astype(np.float32)
    np.testing.assert_allclose(O.merge_partials(m, l, o), O.attention_gqa(k, v, q, qh, L), atol=2e-6, rtol=1e-5)


def test_decode_layer_composition(O):
    """tests/forward_parity_toy.rs:309-386 op order, against float64 numpy."""
    rng = np.random.default_rng(29)
    H, qh, kvh, hd, F, pos = 64, 4, 2, 16, 96, 5
    cfg = O.LayerCfg(H, qh, kvh, hd, F, 0, 0, 1e-5, 10000.0, 1.0)
    w = {n: (rng.standard_normal(s) * 0.1).astype(np.float16) for n, s in
         dict(wq=(qh * hd, H), wk=(kvh * hd, H), wv=(kvh * hd, H), wo=(H, qh * hd), wg=(F, H), wu=(F, H), wd=(H, F)).items()}
    w["attn_norm"] = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    w["ffn_norm"] = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    K = np.zeros((8, kvh, hd), np.float16)
    V = np.zeros((8, kvh, hd), np.float16)
    K[:pos] = rng.standard_normal((pos, kvh, hd)).astype(np.float16)
    V[:pos] = rng.standard_normal((pos, kvh, hd)).astype(np.float16)
    x = rng.standard_normal(H).astype(np.float32)
    K2, V2 = K.copy(), V.copy()
    out, q_rot, att = O.decode_layer(cfg, x, w, K2, V2, pos)
    f = lambda a: a.astype(np.float64)
    xn = f(x) / np.sqrt((f(x) ** 2).mean() + 1e-5) * f(w["attn_norm"])
    q = f(w["wq"]) @ xn
    k = f(w["wk"]) @ xn
    v = f(w["wv"]) @ xn

    def rope64(t, heads):
        t = t.reshape(heads, hd).copy()
        for i in range(hd // 2):
            th = pos * 10000.0 ** (-2.0 * i / hd)
            a, b = t[:, 2 * i].copy(), t[:, 2 * i + 1].copy()
            t[:, 2 * i], t[:, 2 * i + 1] = a * np.cos(th) - b * np.sin(th), a * np.sin(th) + b * np.cos(th)
        return t.ravel()

    q, k = rope64(q, qh), rope64(k, kvh)
    np.testing.assert_allclose(q_rot, q, atol=1e-5)
    Kf, Vf = f(K), f(V)
    Kf[pos] = k.astype(np.float16).reshape(kvh, hd)
    Vf[pos] = v.astype(np.float16).reshape(kvh, hd)
    np.testing.assert_allclose(f(K2[pos]), Kf[pos], atol=2e-3)
    a = np_attention(q.astype(np.float32), K2[:pos + 1], V2[:pos + 1], qh)
    np.testing.assert_allclose(att, a, atol=1e-5)
    x1 = f(x) + f(w["wo"]) @ a
    x1n = x1 / np.sqrt((x1 ** 2).mean() + 1e-5) * f(w["ffn_norm"])
    g, u = f(w["wg"]) @ x1n, f(w["wu"]) @ x1n
    ref = x1 + f(w["wd"]) @ (g / (1 + np.exp(-g)) * u)
    np.testing.assert_allclose(out, ref, atol=2e-5)


def test_prefill_varlen_closed_form(O):
    """Packed causal prefill (tests/attention_prefill_varlen.rs:19-140: 4 / 2 heads, (q_len, kv_len) = (3, 3), (2, 5),
    (1, 4), head_dim 64 and 128, tolerance 1e-6 in the reference) against a float64 restatement; the last q row of a
    sequence equals last-token attention over the same f16-exact keys and values."""
    rng = np.random.default_rng(0)
    for hd in (64, 128):
        qh, kvh = 4, 2
        pairs = [(3, 3), (2, 5), (1, 4)]
        ql = np.array([p[0] for p in pairs], np.uint32)
        kl = np.array([p[1] for p in pairs], np.uint32)
        qo = np.concatenate([[0], np.cumsum(ql)[:-1]]).astype(np.uint32)
        ko = np.concatenate([[0], np.cumsum(kl)[:-1]]).astype(np.uint32)
        q = rng.standard_normal((int(ql.sum()), qh, hd)).astype(np.float32)
        k = rng.standard_normal((int(kl.sum()), kvh, hd)).astype(np.float16).astype(np.float32)
        v = rng.standard_normal((int(kl.sum()), kvh, hd)).astype(np.float16).astype(np.float32)
        out = O.attention_prefill_varlen(q, k, v, qo, ko, ql, kl, qh, kvh, hd)
        for b in range(len(pairs)):
            for i in range(ql[b]):
                for h in range(qh):
                    end = kl[b] - ql[b] + i
                    kk = k[ko[b]:ko[b] + end + 1, h // 2].astype(np.float64)
                    vv = v[ko[b]:ko[b] + end + 1, h // 2].astype(np.float64)
                    s = kk @ q[qo[b] + i, h].astype(np.float64) / np.sqrt(hd)
                    p = np.exp(s - s.max())
                    assert np.abs(out[qo[b] + i, h] - (p / p.sum()) @ vv).max() < 2e-6
            last = O.attention_gqa(k[ko[b]:ko[b] + kl[b]].astype(np.float16), v[ko[b]:ko[b] + kl[b]].astype(np.float16),
                                   q[qo[b] + ql[b] - 1].reshape(-1), qh, int(kl[b]))
            assert np.abs(out[qo[b] + ql[b] - 1].reshape(-1) - last).max() < 2e-6

