"""Packed variable-length prefill attention and the dense -> compressed cache build through the C ABI
(tests/attention_prefill_varlen.rs and tests/forward_with_layer_smoke.rs:332-515 of the reference)."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu


def run_prefill(nat, O, qh, kvh, hd, pairs, seed, sync_form=False):
    rng = np.random.default_rng(seed)
    ql = np.array([p[0] for p in pairs], np.uint32)
    kl = np.array([p[1] for p in pairs], np.uint32)
    qo = np.concatenate([[0], np.cumsum(ql)[:-1]]).astype(np.uint32)
    ko = np.concatenate([[0], np.cumsum(kl)[:-1]]).astype(np.uint32)
    q = rng.standard_normal((int(ql.sum()), qh, hd)).astype(np.float32)
    k = rng.standard_normal((int(kl.sum()), kvh, hd)).astype(np.float32)
    v = rng.standard_normal((int(kl.sum()), kvh, hd)).astype(np.float32)
    dq, dk, dv, do = nat.buf(q), nat.buf(k), nat.buf(v), nat.buf(q.nbytes)
    do.upload(np.full(q.shape, 9.0, np.float32))
    dqo, dko, dql, dkl = nat.buf(qo), nat.buf(ko), nat.buf(ql), nat.buf(kl)
    f = nat.lib.m40llm_attention_prefill_f32_gqa_varlen if sync_form else nat.lib.m40llm_attention_prefill_f32_gqa_varlen_async
    rc = f(nat.ctx, dq.ptr, dk.ptr, dv.ptr, dqo.ptr, dko.ptr, dql.ptr, dkl.ptr, len(pairs), qh, kvh, hd, do.ptr)
    assert rc == 0, rc
    nat.sync(0)
    got = do.download(np.float32, q.shape)
    exp = O.attention_prefill_varlen(q, k, v, qo, ko, ql, kl, qh, kvh, hd)
    return got, exp


@pytest.mark.parametrize("hd", [64, 128])
def test_reference_prefill_case(nat, O, hd):
    """The reference test's batch: (q_len, kv_len) = (3, 3), (2, 5), (1, 4) with 4 / 2 heads."""
    for sync_form in (False, True):
        got, exp = run_prefill(nat, O, 4, 2, hd, [(3, 3), (2, 5), (1, 4)], 11 + hd, sync_form)
        assert_close(got, exp, what=f"prefill hd {hd}")
    nat.free_all()


@pytest.mark.parametrize("qh,kvh,hd,pairs", [
    (8, 2, 64, [(64, 64), (65, 65), (1, 1), (63, 200)]),          # tile boundaries
    (32, 8, 128, [(300, 300), (17, 1000), (128, 129)]),           # Llama-3-8B heads, chunked prefill with a prefix
    (16, 2, 128, [(513, 2048)]),                                  # Qwen heads, long prefix
    (32, 4, 64, [(1000, 1000), (5, 5)]),                          # TinyLlama heads
    (4, 4, 64, [(129, 129)]),                                     # MHA
])
def test_prefill_shapes(nat, O, qh, kvh, hd, pairs):
    got, exp = run_prefill(nat, O, qh, kvh, hd, pairs, qh + hd + len(pairs))
    assert_close(got, exp, what=f"prefill {qh}/{kvh} d{hd} {pairs}")
    nat.free_all()


def test_prefill_full_length_and_last_row_equals_decode(nat, O):
    """Maximum kv length the reference admits (8192), and the last q row of a prefill equals last-token decode
    attention over the same keys and values (after their f16 rounding by the cache)."""
    qh, kvh, hd, L = 8, 2, 128, 8192
    got, exp = run_prefill(nat, O, qh, kvh, hd, [(96, L)], 5)
    assert_close(got, exp, what="prefill kv 8192")
    nat.free_all()


def test_prefill_argument_errors(nat):
    f = nat.lib.m40llm_attention_prefill_f32_gqa_varlen_async
    x = nat.buf(np.zeros(4 * 64 * 8, np.float32))
    one, two, zero, big = (nat.buf(np.array([v], np.uint32)) for v in (1, 2, 0, 9000))
    assert f(nat.ctx, None, x.ptr, x.ptr, zero.ptr, zero.ptr, one.ptr, one.ptr, 1, 4, 2, 64, x.ptr) == -1
    assert f(nat.ctx, x.ptr, x.ptr, x.ptr, zero.ptr, zero.ptr, one.ptr, one.ptr, 0, 4, 2, 64, x.ptr) == -2
    assert f(nat.ctx, x.ptr, x.ptr, x.ptr, zero.ptr, zero.ptr, one.ptr, one.ptr, 1, 3, 2, 64, x.ptr) == -3
    assert f(nat.ctx, x.ptr, x.ptr, x.ptr, zero.ptr, zero.ptr, one.ptr, one.ptr, 1, 4, 2, 32, x.ptr) == -9
    assert f(nat.ctx, x.ptr, x.ptr, x.ptr, zero.ptr, zero.ptr, two.ptr, one.ptr, 1, 4, 2, 64, x.ptr) == -8   # q_len > kv_len
    assert f(nat.ctx, x.ptr, x.ptr, x.ptr, zero.ptr, zero.ptr, zero.ptr, one.ptr, 1, 4, 2, 64, x.ptr) == -8  # q_len == 0
    assert f(nat.ctx, x.ptr, x.ptr, x.ptr, zero.ptr, zero.ptr, one.ptr, big.ptr, 1, 4, 2, 64, x.ptr) == -8   # kv_len > 8192
    nat.free_all()


@pytest.mark.parametrize("kvh,hd,R,bs,L", [(2, 64, 8, 4, 21), (2, 128, 16, 8, 100), (8, 128, 512, 64, 1500), (2, 64, 32, 16, 20)])
def test_build_compressed_from_dense(nat, O, kvh, hd, R, bs, L):
    """Every slot of the compressed cache ends up as token-by-token appends would have left it: bit-exact old K, q4 V
    bytes and scales, ring rows, and lengths; then block-select attention over it matches the oracle."""
    rng = np.random.default_rng(L + hd)
    slots, max_seq = 3, L + 4
    dense = nat.kv_dense(max_seq, slots, kvh, hd)
    comp = nat.kv_compressed(max_seq, slots, kvh, hd, R, bs, 3)
    ks = rng.standard_normal((slots, L, kvh, hd)).astype(np.float16)
    vs = rng.standard_normal((slots, L, kvh, hd)).astype(np.float16)
    for s in range(slots):
        nat.kv_fill(dense, s, ks[s], vs[s])
    assert nat.lib.m40llm_kvcache_build_compressed_from_dense(nat.ctx, comp, dense, L) == 0
    old_len = max(L - R, 0)
    for s in range(slots):
        old_k, q4, sc, rk, rv = O.compressed_state_from_dense(ks[s], vs[s], L, R)
        for t in sorted({0, old_len // 2, old_len - 1} & set(range(old_len))):
            k = np.empty((kvh, hd), np.float16)
            b = np.empty((kvh, hd // 2), np.uint8)
            f = np.empty(kvh, np.float32)
            assert nat.lib.m40llm_kvcache_debug_read_old_token(nat.ctx, comp, s, t, k.ctypes.data_as(C.c_void_p),
                                                               b.ctypes.data_as(C.c_void_p), f.ctypes.data_as(C.c_void_p)) == 0
            assert np.array_equal(k.view(np.uint16), old_k[t].view(np.uint16))
            assert np.array_equal(b, q4[t]) and np.array_equal(f, sc[t])
        q = rng.standard_normal(8 * hd).astype(np.float32)
        dq, do = nat.buf(q), nat.buf(q.nbytes)
        rc = nat.lib.m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async(
            nat.ctx, comp, s, dq.ptr, 8, L, R, bs, 3, do.ptr)
        assert rc == 0, rc
        nat.sync(1)
        exp, *_ = O.attention_compressed(old_k, q4, sc, rk, rv, q, 8, L, R, bs, 3)
        assert_close(do.download(np.float32, q.shape), exp, what=f"slot {s} attention over the built cache")
    # argument errors of the reference
    assert nat.lib.m40llm_kvcache_build_compressed_from_dense(nat.ctx, dense, dense, L) == -2
    assert nat.lib.m40llm_kvcache_build_compressed_from_dense(nat.ctx, comp, dense, max_seq + 1) == -4
    other = nat.kv_dense(max_seq, slots, kvh + 1, hd)
    assert nat.lib.m40llm_kvcache_build_compressed_from_dense(nat.ctx, comp, other, L) == -3
    for kv in (dense, comp, other):
        nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()
