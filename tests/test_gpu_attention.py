"""Dense decode attention through the C ABI against the oracle (the reference's CPU attention restated).
Mirrors tests/attention_parity_cuda_grid.rs (MHA grid, GQA grid, long hd64) and
tests/attention_batched_varlen.rs; tolerance |a-e| <= 1e-3 + 2e-3|e| (the reference uses 1e-3 absolute)."""
import numpy as np
import pytest

from helpers import assert_close
from test_oracle_kat import closed_form_kv

pytestmark = pytest.mark.gpu


def run_gqa(nat, kv, seq, q, qh, L):
    dq, do = nat.buf(q), nat.buf(q.nbytes)
    rc = nat.lib.m40llm_attention_last_token_f32_gqa_async(nat.ctx, kv, seq, dq.ptr, qh, L, do.ptr)
    assert rc == 0, rc
    nat.sync(1)
    return do.download(np.float32, q.shape)


@pytest.mark.parametrize("heads", [1, 2, 3, 4])
def test_mha_grid_closed_form(nat, O, heads):
    """tests/attention_parity_cuda_grid.rs MHA grid with the closed-form K/V/q of the CPU grid."""
    for hd in (1, 5, 7, 8, 16, 31, 32, 63, 64):
        dim = heads * hd
        kv = nat.kv_dense(16, 1, heads, hd)
        k, v, q = closed_form_kv(16, dim)
        for t in range(16):
            dk, dv = nat.buf(k[t]), nat.buf(v[t])
            assert nat.lib.m40llm_kvcache_append_token_f32_async(nat.ctx, kv, 0, dk.ptr, dv.ptr) == 0
        nat.sync(1)
        k16, v16 = O.f32_to_f16(k).reshape(16, heads, hd), O.f32_to_f16(v).reshape(16, heads, hd)
        for L in (1, 2, 3, 4, 7, 8, 16):
            dq, do = nat.buf(q), nat.buf(q.nbytes)
            assert nat.lib.m40llm_attention_last_token_f32(nat.ctx, kv, 0, dq.ptr, L, do.ptr) == 0
            assert_close(do.download(np.float32, dim), O.attention_gqa(k16, v16, q, heads, L), what=f"mha h{heads} d{hd} L{L}")
        nat.lib.m40llm_kvcache_destroy(kv)
        nat.free_all()


@pytest.mark.parametrize("qh,kvh", [(2, 1), (4, 1), (8, 2), (32, 4), (32, 8), (16, 2), (12, 2)])
@pytest.mark.parametrize("hd", [1, 5, 8, 16, 32, 64, 128, 256])
def test_gqa_grid(nat, O, qh, kvh, hd):
    rng = np.random.default_rng(qh * 7 + hd)
    max_seq = 700
    kv = nat.kv_dense(max_seq, 2, kvh, hd)
    k = rng.standard_normal((max_seq, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((max_seq, kvh, hd)).astype(np.float16)
    nat.kv_fill(kv, 1, k, v)
    for L in (1, 2, 17, 64, 65, 128, 300, 700):
        q = rng.standard_normal(qh * hd).astype(np.float32)
        got = run_gqa(nat, kv, 1, q, qh, L)
        assert_close(got, O.attention_gqa(k, v, q, qh, L), what=f"gqa {qh}/{kvh} d{hd} L{L}")
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("qh,kvh,hd,L", [(8, 2, 64, 256), (32, 4, 64, 2048), (32, 8, 128, 8192), (16, 2, 128, 4096),
                                          (32, 8, 128, 16384), (32, 4, 64, 12345)])
def test_config_shapes(nat, O, qh, kvh, hd, L):
    """BASELINE configs: toy (8/2/64 @256), TinyLlama (32/4/64 @2048), Llama-3-8B (32/8/128), Qwen (16/2/128)."""
    rng = np.random.default_rng(L)
    kv = nat.kv_dense(L, 1, kvh, hd)
    k = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    nat.kv_fill(kv, 0, k, v)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    got = run_gqa(nat, kv, 0, q, qh, L)
    assert_close(got, O.attention_gqa(k, v, q, qh, L), what=f"{qh}/{kvh}/{hd} L{L}")
    # seq_len read from device memory (graph-replay variant) and the synchronous variant agree bit for bit
    dq, do, dl = nat.buf(q), nat.buf(q.nbytes), nat.buf(np.array([L], np.uint32))
    assert nat.lib.m40llm_attention_last_token_f32_gqa_seq_len_dev_async(nat.ctx, kv, 0, dq.ptr, qh, dl.ptr, do.ptr) == 0
    nat.sync(1)
    assert_close(do.download(np.float32, q.shape), got, what="seq_len_dev")
    assert nat.lib.m40llm_attention_last_token_f32_gqa(nat.ctx, kv, 0, dq.ptr, qh, L, do.ptr) == 0
    assert np.array_equal(do.download(np.float32, q.shape), got)
    # split-K: partial triples over token ranges merge to the same output
    bounds = [0, L // 3, L // 3, (2 * L) // 3 + 1, L]
    parts = len(bounds) - 1
    dm, dl_, dop = nat.buf(parts * qh * 4), nat.buf(parts * qh * 4), nat.buf(parts * qh * hd * 4)
    for r in range(parts):
        rc = nat.lib.m40llm_attention_last_token_f32_gqa_partial_async(
            nat.ctx, kv, 0, dq.ptr, qh, bounds[r], bounds[r + 1], dm.ptr + r * qh * 4, dl_.ptr + r * qh * 4,
            dop.ptr + r * qh * hd * 4)
        assert rc == 0, rc
    assert nat.lib.m40llm_attention_merge_partials_async(nat.ctx, dm.ptr, dl_.ptr, dop.ptr, parts, qh, hd, do.ptr) == 0
    nat.sync(1)
    assert_close(do.download(np.float32, q.shape), O.attention_gqa(k, v, q, qh, L), what="split-K merge")
    m = dm.download(np.float32, (parts, qh))
    l = dl_.download(np.float32, (parts, qh))
    o = dop.download(np.float32, (parts, qh, hd))
    assert np.all(l[1] == 0)  # the empty range contributes nothing
    assert_close(O.merge_partials(m, l, o), O.attention_gqa(k, v, q, qh, L), what="oracle merge of device partials")
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("qh,kvh,hd,lens", [(4, 2, 64, [1, 3, 5]), (32, 8, 128, [512, 8192, 77, 4096, 1, 2049]),
                                            (32, 4, 64, [1024, 16, 384, 768]), (16, 2, 128, [33] * 9)])
def test_batched_varlen(nat, O, qh, kvh, hd, lens):
    """tests/attention_batched_varlen.rs:36-71, 200-221: batched == per-sequence, any slot order."""
    rng = np.random.default_rng(len(lens) + hd)
    B, max_seq = len(lens), max(lens)
    slots = B + 2
    kv = nat.kv_dense(max_seq, slots, kvh, hd)
    ids = rng.permutation(slots)[:B].astype(np.uint32)
    K = np.zeros((slots, max_seq, kvh, hd), np.float16)
    V = np.zeros((slots, max_seq, kvh, hd), np.float16)
    for b in range(B):
        K[ids[b], :lens[b]] = rng.standard_normal((lens[b], kvh, hd)).astype(np.float16)
        V[ids[b], :lens[b]] = rng.standard_normal((lens[b], kvh, hd)).astype(np.float16)
        nat.kv_fill(kv, int(ids[b]), K[ids[b], :lens[b]], V[ids[b], :lens[b]])
    q = rng.standard_normal((B, qh, hd)).astype(np.float32)
    dq, do = nat.buf(q), nat.buf(q.nbytes)
    dids, dlens = nat.buf(ids), nat.buf(np.array(lens, np.uint32))
    assert nat.lib.m40llm_attention_last_token_f32_gqa_batched_async(nat.ctx, kv, dids.ptr, dlens.ptr, B, dq.ptr, qh, do.ptr) == 0
    nat.sync(1)
    got = do.download(np.float32, q.shape)
    assert_close(got, O.attention_gqa_batched(K, V, ids, np.array(lens, np.uint32), q, qh), what="batched")
    for b in range(B):
        one = run_gqa(nat, kv, int(ids[b]), q[b].ravel().copy(), qh, lens[b])
        # the two calls split the tokens into different chunks, so P is rounded to f16 against different running
        # maxima: equal within the parity tolerance, not bit for bit
        assert_close(got[b].ravel(), one, what=f"batched row {b} vs single")
    assert nat.lib.m40llm_attention_last_token_f32_gqa_batched(nat.ctx, kv, dids.ptr, dlens.ptr, B, dq.ptr, qh, do.ptr) == 0
    assert np.array_equal(do.download(np.float32, q.shape), got)
    # a row with a zero length or an out-of-range id is rejected (rc -8 in the reference, kernels.cu:4737-4747)
    bad = np.array(lens, np.uint32)
    bad[0] = 0
    dbad = nat.buf(bad)
    assert nat.lib.m40llm_attention_last_token_f32_gqa_batched(nat.ctx, kv, dids.ptr, dbad.ptr, B, dq.ptr, qh, do.ptr) == -8
    assert nat.lib.m40llm_attention_last_token_f32_gqa_batched(nat.ctx, kv, dids.ptr, dlens.ptr, 0, dq.ptr, qh, do.ptr) == -2
    assert nat.lib.m40llm_attention_last_token_f32_gqa_batched(nat.ctx, kv, dids.ptr, dlens.ptr, B, dq.ptr, qh + 1, do.ptr) == -3
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_argument_errors(nat):
    kv = nat.kv_dense(8, 2, 2, 64)
    q = nat.buf(np.zeros(8 * 64, np.float32))
    L = nat.lib
    assert L.m40llm_attention_last_token_f32_gqa_async(nat.ctx, kv, 0, None, 8, 1, q.ptr) == -1
    assert L.m40llm_attention_last_token_f32_gqa_async(nat.ctx, kv, 2, q.ptr, 8, 1, q.ptr) == -2
    assert L.m40llm_attention_last_token_f32_gqa_async(nat.ctx, kv, 0, q.ptr, 8, 0, q.ptr) == -3
    assert L.m40llm_attention_last_token_f32_gqa_async(nat.ctx, kv, 0, q.ptr, 8, 9, q.ptr) == -3
    assert L.m40llm_attention_last_token_f32_gqa_async(nat.ctx, kv, 0, q.ptr, 3, 1, q.ptr) == -6
    assert L.m40llm_attention_last_token_f32(nat.ctx, kv, 0, q.ptr, 0, q.ptr) == -3
    assert L.m40llm_attention_last_token_f32_gqa_dense_recent_async(nat.ctx, kv, 0, q.ptr, 8, 4, 2, q.ptr) == -100
    L.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("max_seq,hd", [(64, 64), (4096, 128), (2048, 48)])
def test_batched_async_rejected_row_is_zero_and_flagged(nat, O, max_seq, hd):
    """The async batched call cannot return a per-row code: a row whose length or slot is out of range reads no
    cache data, raises status bit 1 and gets a zero output row whether the launch uses one split (short cache), many
    (long cache) or the generic kernel (head_dim 48); the other rows are unaffected. The output buffer is poisoned
    first and the arena is dirtied by a previous call so that stale partials would show."""
    rng = np.random.default_rng(max_seq)
    qh, kvh, B = 8, 2, 4
    kv = nat.kv_dense(max_seq, B, kvh, hd)
    lens = np.array([max_seq, 17, max_seq - 3, 5], np.uint32)
    K = np.zeros((B, max_seq, kvh, hd), np.float16)
    V = np.zeros((B, max_seq, kvh, hd), np.float16)
    for b in range(B):
        K[b, :lens[b]] = rng.standard_normal((lens[b], kvh, hd)).astype(np.float16)
        V[b, :lens[b]] = rng.standard_normal((lens[b], kvh, hd)).astype(np.float16)
        nat.kv_fill(kv, b, K[b, :lens[b]], V[b, :lens[b]])
    q = rng.standard_normal((B, qh, hd)).astype(np.float32)
    ids = np.arange(B, dtype=np.uint32)
    dq, do, dids, dlens = nat.buf(q), nat.buf(q.nbytes), nat.buf(ids), nat.buf(lens)
    f = nat.lib.m40llm_attention_last_token_f32_gqa_batched_async
    assert f(nat.ctx, kv, dids.ptr, dlens.ptr, B, dq.ptr, qh, do.ptr) == 0  # fills the partial arena with real data
    nat.sync(1)
    good = do.download(np.float32, q.shape)
    assert_close(good, O.attention_gqa_batched(K, V, ids, lens, q, qh), what="clean batch")
    for bad_row, bad_len, bad_id in ((2, max_seq + 1, 2), (0, 0, 0), (1, 17, B + 3)):
        l2, i2 = lens.copy(), ids.copy()
        l2[bad_row], i2[bad_row] = bad_len, bad_id
        dlens.upload(l2)
        dids.upload(i2)
        do.upload(np.full(q.shape, 7.0, np.float32))
        assert f(nat.ctx, kv, dids.ptr, dlens.ptr, B, dq.ptr, qh, do.ptr) == 0
        st = np.zeros(1, np.uint32)
        assert nat.lib.m40llm_context_take_device_status(nat.ctx, st.ctypes.data) == 0 and st[0] == 1
        got = do.download(np.float32, q.shape)
        assert np.all(got[bad_row] == 0.0), f"rejected row {bad_row} not zero"
        keep = [b for b in range(B) if b != bad_row]
        assert np.array_equal(got[keep], good[keep])
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()
