"""KV cache append / read-back through the C ABI (tests/kv_f32_to_f16_append.rs, tests/kv_layout.rs and the
ring-wrap test tests/attention_parity_cuda_grid.rs:1130-1355 of the reference). Integer/byte results are bit-exact."""
import ctypes as C

import numpy as np
import pytest

from helpers import rope_rows_np

pytestmark = pytest.mark.gpu


def read_token(nat, kv, seq, t, kvh, hd):
    k = np.empty((kvh, hd), np.float16)
    v = np.empty((kvh, hd), np.float16)
    rc = nat.lib.m40llm_kvcache_debug_read_token(nat.ctx, kv, seq, t, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p))
    assert rc == 0, rc
    return k, v


def read_old(nat, kv, seq, t, kvh, hd):
    k = np.empty((kvh, hd), np.float16)
    q4 = np.empty((kvh, hd // 2), np.uint8)
    sc = np.empty(kvh, np.float32)
    rc = nat.lib.m40llm_kvcache_debug_read_old_token(nat.ctx, kv, seq, t, k.ctypes.data_as(C.c_void_p),
                                                     q4.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p))
    assert rc == 0, rc
    return k, q4, sc


@pytest.mark.parametrize("kvh,hd", [(3, 5), (2, 64), (8, 128)])
def test_append_f32_is_f16_rounding(nat, O, kvh, hd):
    rng = np.random.default_rng(kvh + hd)
    kv = nat.kv_dense(8, 2, kvh, hd)
    ks = rng.standard_normal((4, kvh * hd)).astype(np.float32)
    vs = rng.standard_normal((4, kvh * hd)).astype(np.float32) * 100
    for t in range(4):
        dk, dv = nat.buf(ks[t]), nat.buf(vs[t])
        assert nat.lib.m40llm_kvcache_append_token_f32_async(nat.ctx, kv, 1, dk.ptr, dv.ptr) == 0
    nat.sync(1)
    for t in range(4):
        k, v = read_token(nat, kv, 1, t, kvh, hd)
        assert np.array_equal(k.view(np.uint16).ravel(), O.f32_to_f16(ks[t]).view(np.uint16))
        assert np.array_equal(v.view(np.uint16).ravel(), O.f32_to_f16(vs[t]).view(np.uint16))
    # sequence 0 untouched; f16 append variant; capacity and argument errors
    k0, _ = read_token(nat, kv, 0, 0, kvh, hd)
    assert not k0.view(np.uint16).any()
    h = nat.buf(ks[0].astype(np.float16))
    assert nat.lib.m40llm_kvcache_append_token(nat.ctx, kv, 0, h.ptr, h.ptr) == 0
    k0, v0 = read_token(nat, kv, 0, 0, kvh, hd)
    assert np.array_equal(k0.ravel(), ks[0].astype(np.float16)) and np.array_equal(v0.ravel(), ks[0].astype(np.float16))
    assert nat.lib.m40llm_kvcache_append_token_f32_async(nat.ctx, kv, 2, h.ptr, h.ptr) == -2
    for _ in range(4):
        assert nat.lib.m40llm_kvcache_append_token_f32(nat.ctx, kv, 1, dk.ptr, dv.ptr) == 0
    assert nat.lib.m40llm_kvcache_append_token_f32_async(nat.ctx, kv, 1, dk.ptr, dv.ptr) == -4
    assert nat.lib.m40llm_kvcache_debug_read_token(nat.ctx, kv, 0, 8, None, None) == -1
    assert nat.lib.m40llm_kvcache_reset(nat.ctx, kv) == 0
    assert nat.lib.m40llm_kvcache_append_token_f32(nat.ctx, kv, 1, dk.ptr, dv.ptr) == 0
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("kvh,hd,base", [(4, 64, 1e4), (8, 128, 5e5), (2, 128, 1e6)])
def test_fused_rope_append_equals_separate_ops(nat, O, layout, kvh, hd, base):
    """tests/kv_f32_to_f16_append.rs:128-245: fused RoPE(K)+cast+append == rope then f16 cast."""
    rng = np.random.default_rng(hd + layout)
    kv = nat.kv_dense(4200, 1, kvh, hd)
    positions = [0, 1, 77, 4100]
    for pos in positions:
        k = rng.standard_normal(kvh * hd).astype(np.float32)
        v = rng.standard_normal(kvh * hd).astype(np.float32)
        dk, dv = nat.buf(k), nat.buf(v)
        assert nat.lib.m40llm_kvcache_append_token_f32_rope_k_at_layout_async(nat.ctx, kv, 0, dk.ptr, dv.ptr, pos, 999,
                                                                              base, 1.0, layout) == 0
        nat.sync(1)
        gk, gv = read_token(nat, kv, 0, pos, kvh, hd)
        # the separate op on the device (rope in place) then f16 must agree bit for bit
        assert nat.lib.m40llm_rope_f32_inplace_layout_async(nat.ctx, dk.ptr, 1, kvh, hd, pos, base, 1.0, layout) == 0
        nat.sync(1)
        sep = dk.download(np.float32, kvh * hd)
        assert np.array_equal(gk.view(np.uint16).ravel(), O.f32_to_f16(sep).view(np.uint16))
        assert np.array_equal(gv.view(np.uint16).ravel(), O.f32_to_f16(v).view(np.uint16))
        ek = O.rope(k, kvh, hd, pos, base, 1.0, layout)
        np.testing.assert_allclose(gk.astype(np.float32).ravel(), ek, atol=3e-3)
        dpos = nat.buf(np.array([pos], np.uint32))
        dk.upload(k)
        assert nat.lib.m40llm_kvcache_append_token_f32_rope_k_position_dev_layout_async(
            nat.ctx, kv, 0, dk.ptr, dv.ptr, dpos.ptr, base, 1.0, layout) == 0
        nat.sync(1)
        gk2, _ = read_token(nat, kv, 0, pos, kvh, hd)
        assert np.array_equal(gk2, gk)
    assert nat.lib.m40llm_kvcache_append_token_f32_rope_k_at_layout_async(nat.ctx, kv, 0, dk.ptr, dv.ptr, 4200, 0, base,
                                                                          1.0, layout) == -5
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("kvh,hd,R,bs,L", [(2, 64, 4, 4, 16), (2, 128, 4, 32, 5), (2, 128, 8, 4, 30), (4, 64, 16, 8, 16)])
def test_compressed_append_lifecycle(nat, O, kvh, hd, R, bs, L):
    """Token-by-token appends leave exactly the state of cuda/kernels.cu:6108-6250: old K = f16 K, old V = q4 of the
    f16 V that sat in the ring, newest min(L, R) tokens in ring slot t % R; and the bulk loader builds the same state."""
    rng = np.random.default_rng(R * 100 + L)
    k = rng.standard_normal((L, kvh, hd)).astype(np.float32)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float32)
    k16, v16 = O.f32_to_f16(k), O.f32_to_f16(v)
    old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k16, v16, L, R)
    kv = nat.kv_compressed(L, 2, kvh, hd, R, bs, 3)
    nat.kv_append_tokens(kv, 1, k.reshape(L, -1), v.reshape(L, -1), scale=0.0)
    kv2 = nat.kv_compressed(L, 2, kvh, hd, R, bs, 3)
    nat.kv_fill(kv2, 1, k16, v16, final_len=L)
    for cache in (kv, kv2):
        for t in range(max(L - R, 0)):
            gk, gq, gs = read_old(nat, cache, 1, t, kvh, hd)
            assert np.array_equal(gk.view(np.uint16), old_k[t].view(np.uint16))
            assert np.array_equal(gq, q4[t])
            assert np.array_equal(gs.view(np.uint32), sc[t].view(np.uint32))
        seq_len = C.c_uint32()
        nblk = max((max(L - R, 0) + bs - 1) // bs, 1)
        counts = np.zeros(nblk, np.uint32)
        grk = np.empty((R, kvh, hd), np.float16)
        grv = np.empty((R, kvh, hd), np.float16)
        junk = [np.zeros(nblk * kvh * hd, np.float32) for _ in range(2)] + [np.zeros(nblk * kvh * hd, np.float16) for _ in range(2)]
        p = lambda a: a.ctypes.data_as(C.c_void_p)
        rc = nat.lib.m40llm_kvcache_debug_read_compressed_state(nat.ctx, cache, 1, C.byref(seq_len), p(counts), p(grk), p(grv),
                                                                p(junk[0]), p(junk[1]), p(junk[2]), p(junk[3]), None, None, None)
        assert rc == 0, rc
        assert seq_len.value == L
        assert np.array_equal(grk.view(np.uint16), rk.view(np.uint16)) and np.array_equal(grv.view(np.uint16), rv.view(np.uint16))
        assert counts.sum() == max(L - R, 0)
    assert nat.lib.m40llm_kvcache_reset(nat.ctx, kv) == 0
    gk, gq, gs = read_old(nat, kv, 1, 0, kvh, hd)
    assert not gk.view(np.uint16).any() and not gq.any() and not gs.any()
    for cache in (kv, kv2):
        nat.lib.m40llm_kvcache_destroy(cache)
    nat.free_all()


def test_compressed_rope_append_uses_position(nat, O):
    rng = np.random.default_rng(2)
    kvh, hd, R = 2, 128, 4
    kv = nat.kv_compressed(64, 1, kvh, hd, R, 8, 2)
    k = rng.standard_normal((10, kvh * hd)).astype(np.float32)
    v = rng.standard_normal((10, kvh * hd)).astype(np.float32)
    nat.kv_append_tokens(kv, 0, k, v, base=1e6, scale=1.0, layout=1)
    for t in range(6):
        gk, _, _ = read_old(nat, kv, 0, t, kvh, hd)
        ek = O.rope(k[t], kvh, hd, t, 1e6, 1.0, 1).reshape(kvh, hd)
        np.testing.assert_allclose(gk.astype(np.float32), ek, atol=3e-3)
    # unsupported configurations are refused at creation
    assert not nat.lib.m40llm_kvcache_create_compressed(nat.ctx, 64, 1, kvh, 32, R, 8, 2, 0, 0, 2)
    assert not nat.lib.m40llm_kvcache_create_compressed(nat.ctx, 64, 1, kvh, hd, 0, 8, 2, 0, 0, 2)
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()
