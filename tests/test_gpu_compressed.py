"""Block-select attention (FP16 K + q4 V + ring, and the dense-backed form) through the C ABI against the oracle.
Mirrors tests/attention_parity_cuda_grid.rs:182-843, 1130-1355. Selected block indices are compared exactly,
except where the exact scores tie within 1e-6 at the cut-off; outputs within 1e-3 + 2e-3|e|."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close, assert_selection_matches

pytestmark = pytest.mark.gpu


def build_state(nat, O, rng, kvh, hd, L, R, bs, top, max_seq=None, slots=1, seq=0):
    k = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    kv = nat.kv_compressed(max_seq or L, slots, kvh, hd, R, bs, top)
    nat.kv_fill(kv, seq, k, v, final_len=L)
    return kv, k, v, O.compressed_state_from_dense(k, v, L, R)


def run_direct(nat, kv, seq, q, qh, L, R, bs, top):
    dq, do = nat.buf(q), nat.buf(q.nbytes)
    rc = nat.lib.m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async(
        nat.ctx, kv, seq, dq.ptr, qh, L, R, bs, top, do.ptr)
    assert rc == 0, rc
    nat.sync(1)
    sel = np.empty((qh, 64), np.uint32)
    sc = np.empty((qh, 64), np.float32)
    assert nat.lib.m40llm_kvcache_debug_last_selected_blocks(nat.ctx, qh, sel.ctypes.data_as(C.c_void_p),
                                                             sc.ctypes.data_as(C.c_void_p)) == 0
    return do.download(np.float32, q.shape), sel, sc


def check_selection(O, old_k, q, qh, kvh, hd, old_len, bs, top, sel, sel_scores, what):
    g = qh // kvh
    for h in range(qh):
        blocks, bsc, s32, s64 = O.block_select_head(old_k, q[h * hd:(h + 1) * hd], h // g, old_len, bs, top)
        got = [int(b) for b in sel[h] if b != 0xFFFFFFFF]
        assert_selection_matches(got, blocks, s64, what=f"{what} head {h}")
        gs = sel_scores[h, :len(got)]
        assert np.all(np.diff(gs) <= 0), f"{what} head {h}: scores not descending"
        np.testing.assert_allclose(gs, [s64[b] for b in got], atol=2e-5)


@pytest.mark.parametrize("qh,kvh,hd,L,R,bs,top", [
    (4, 2, 64, 16, 4, 4, 3),       # all old blocks selected (reference test :216-306)
    (4, 2, 128, 5, 4, 32, 8),      # one partial old block (:618-673)
    (4, 2, 128, 70, 6, 8, 64),     # hd128, all selected (:736-794)
    (8, 2, 64, 3, 4, 4, 2),        # seq_len < recent window: ring only
    (8, 2, 64, 4, 4, 4, 2),        # seq_len == recent window
    (32, 4, 64, 1500, 128, 32, 16),
    (16, 2, 128, 3000, 512, 64, 8),
    (32, 8, 128, 2049, 1024, 32, 8),  # the reference's default config (kv_compression.rs:85-98)
    (16, 2, 128, 777, 100, 7, 5),     # odd block size and window, partial last block
])
def test_direct_q4_attention(nat, O, qh, kvh, hd, L, R, bs, top):
    rng = np.random.default_rng(L * 3 + R)
    kv, k, v, (old_k, q4, sc, rk, rv) = build_state(nat, O, rng, kvh, hd, L, R, bs, top)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    got, sel, sel_sc = run_direct(nat, kv, 0, q, qh, L, R, bs, top)
    exp, esel, ecnt, _ = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, L, R, bs, top)
    check_selection(O, old_k, q, qh, kvh, hd, max(L - R, 0), bs, top, sel, sel_sc, f"L{L}")
    assert_close(got, exp, what=f"q4 direct {qh}/{kvh}/{hd} L{L} R{R} bs{bs} top{top}")
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_ring_wrap_after_many_appends(nat, O):
    """tests/attention_parity_cuda_grid.rs:1130-1355: append past several ring wraps token by token, attend at
    several lengths on the way."""
    rng = np.random.default_rng(5)
    qh, kvh, hd, R, bs, top, L = 8, 2, 64, 8, 4, 3, 45
    k = rng.standard_normal((L, kvh, hd)).astype(np.float32)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float32)
    k16, v16 = O.f32_to_f16(k), O.f32_to_f16(v)
    kv = nat.kv_compressed(64, 1, kvh, hd, R, bs, top)
    done = 0
    for upto in (7, 8, 9, 17, 33, 45):
        nat.kv_append_tokens(kv, 0, k[done:upto].reshape(upto - done, -1), v[done:upto].reshape(upto - done, -1), start=done)
        done = upto
        q = rng.standard_normal(qh * hd).astype(np.float32)
        got, sel, sel_sc = run_direct(nat, kv, 0, q, qh, upto, R, bs, top)
        old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k16, v16, upto, R)
        exp, *_ = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, upto, R, bs, top)
        check_selection(O, old_k, q, qh, kvh, hd, max(upto - R, 0), bs, top, sel, sel_sc, f"wrap {upto}")
        assert_close(got, exp, what=f"ring wrap at {upto}")
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_selection_ties_and_nan(nat, O):
    """Ties go to the lower block index; NaN-scored blocks are never selected (kernels.cu:2913-2927)."""
    rng = np.random.default_rng(6)
    qh, kvh, hd, R, bs, top = 2, 1, 64, 4, 8, 3
    base = rng.standard_normal((bs, kvh, hd)).astype(np.float16)
    k = np.concatenate([np.tile(base, (6, 1, 1)), rng.standard_normal((R, kvh, hd)).astype(np.float16)])
    L = k.shape[0]
    v = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    kv = nat.kv_compressed(L, 1, kvh, hd, R, bs, top)
    nat.kv_fill(kv, 0, k, v, final_len=L)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    _, sel, _ = run_direct(nat, kv, 0, q, qh, L, R, bs, top)
    for h in range(qh):
        assert sorted(int(b) for b in sel[h, :3]) == [0, 1, 2]
    k[bs:2 * bs, 0, 0] = np.float16(np.nan)
    nat.kv_fill(kv, 0, k, v, final_len=L)
    got, sel, _ = run_direct(nat, kv, 0, q, qh, L, R, bs, 6)
    for h in range(qh):
        chosen = [int(b) for b in sel[h] if b != 0xFFFFFFFF]
        assert 1 not in chosen and len(chosen) == 5
    assert np.all(np.isfinite(got))
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


@pytest.mark.parametrize("qh,kvh,hd,L,R,bs,top", [(4, 2, 64, 16, 4, 4, 3), (32, 4, 64, 1200, 256, 32, 16), (16, 2, 128, 900, 64, 16, 6)])
def test_dense_backed_block_select(nat, O, qh, kvh, hd, L, R, bs, top):
    """m40llm_attention_last_token_f32_gqa_block_select_exact_async (kernels.cu:4025-4070) over a dense cache."""
    rng = np.random.default_rng(L)
    k = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((L, kvh, hd)).astype(np.float16)
    kv = nat.kv_dense(L, 1, kvh, hd)
    nat.kv_fill(kv, 0, k, v)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    dq, do = nat.buf(q), nat.buf(q.nbytes)
    assert nat.lib.m40llm_attention_last_token_f32_gqa_block_select_exact_async(nat.ctx, kv, 0, dq.ptr, qh, L, R, bs, top, do.ptr) == 0
    nat.sync(1)
    assert_close(do.download(np.float32, q.shape), O.attention_block_select_dense(k, v, q, qh, L, R, bs, top), what="dense-backed")
    if top * bs >= L - R:  # every old block selected: equals plain dense attention (reference test :452-486)
        assert_close(do.download(np.float32, q.shape), O.attention_gqa(k, v, q, qh, L), what="== dense")
    # host-visible selection of q head 0 (kernels.cu:6449-6677)
    blocks = np.zeros(64, np.uint32); scores = np.zeros(64, np.float32); st = np.zeros(64, np.uint32); en = np.zeros(64, np.uint32)
    cnt, total = C.c_uint32(), C.c_uint32()
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    rc = nat.lib.m40llm_kvcache_debug_select_old_blocks(nat.ctx, kv, 0, dq.ptr, qh, L, R, bs, top, p(blocks), p(scores), p(st), p(en),
                                                        C.byref(cnt), 64, C.byref(total))
    assert rc == 0, rc
    eb, es, s32, s64 = O.block_select_head(k, q[:hd], 0, L - R, bs, top)
    assert total.value == (L - R + bs - 1) // bs and cnt.value == len(eb)
    assert_selection_matches(blocks[:cnt.value], eb, s64, what="debug_select")
    assert np.array_equal(st[:cnt.value], blocks[:cnt.value] * bs)
    assert np.array_equal(en[:cnt.value], np.minimum(st[:cnt.value] + bs, L - R))
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_qwen_long_context_shape(nat, O):
    """BASELINE config 3 at full size: Qwen2.5-3B heads (16/2/128), context 32768, block 64, top 64, recent 512."""
    rng = np.random.default_rng(33)
    qh, kvh, hd, L, R, bs, top = 16, 2, 128, 32768, 512, 64, 64
    kv, k, v, (old_k, q4, sc, rk, rv) = build_state(nat, O, rng, kvh, hd, L, R, bs, top)
    q = rng.standard_normal(qh * hd).astype(np.float32)
    got, sel, sel_sc = run_direct(nat, kv, 0, q, qh, L, R, bs, top)
    exp, esel, ecnt, union = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, L, R, bs, top)
    check_selection(O, old_k, q, qh, kvh, hd, L - R, bs, top, sel, sel_sc, "qwen 32k")
    assert_close(got, exp, what="qwen 32k")
    assert top * bs * kvh <= union <= top * bs * qh
    # split-K over 4 ranks' block ranges: score exchange, global top-k, partial attention, merge
    nb = (L - R + bs - 1) // bs
    P = 4
    bounds = [r * nb // P for r in range(P + 1)]
    dq = nat.buf(q)
    scores = np.empty((qh, nb), np.float32)
    for r in range(P):
        n = bounds[r + 1] - bounds[r]
        ds = nat.buf(qh * n * 4)
        assert nat.lib.m40llm_kvcache_score_old_blocks_async(nat.ctx, kv, 0, dq.ptr, qh, L, bounds[r], bounds[r + 1], ds.ptr) == 0
        nat.sync(1)
        scores[:, bounds[r]:bounds[r + 1]] = ds.download(np.float32, (qh, n))
    glob = np.full((qh, 64), 0xFFFFFFFF, np.uint32)
    for h in range(qh):
        order = sorted(range(nb), key=lambda b: (-scores[h, b], b))[:top]
        glob[h, :len(order)] = order
        _, _, _, s64 = O.block_select_head(old_k, q[h * hd:(h + 1) * hd], h // (qh // kvh), L - R, bs, top)
        assert_selection_matches(order, [int(b) for b in esel[h, :ecnt[h]]], s64, what=f"split-K global top-k head {h}")
    dblk = nat.buf(glob)
    dm, dl, dop, do = nat.buf(P * qh * 4), nat.buf(P * qh * 4), nat.buf(P * qh * hd * 4), nat.buf(q.nbytes)
    for r in range(P):
        rc = nat.lib.m40llm_attention_compressed_selected_partial_async(
            nat.ctx, kv, 0, dq.ptr, qh, L, dblk.ptr, bounds[r], bounds[r + 1], 1 if r == P - 1 else 0,
            dm.ptr + r * qh * 4, dl.ptr + r * qh * 4, dop.ptr + r * qh * hd * 4)
        assert rc == 0, rc
    assert nat.lib.m40llm_attention_merge_partials_async(nat.ctx, dm.ptr, dl.ptr, dop.ptr, P, qh, hd, do.ptr) == 0
    nat.sync(1)
    assert_close(do.download(np.float32, q.shape), exp, what="compressed split-K merge")
    # the same exchange with the selection on the device: local top-k (score, block) pairs per rank, the "gathered"
    # pair array, the global list, triples as one message per rank, the gathered merge; no host step in between
    for P2 in (1, 3, 8):
        b2 = [r * nb // P2 for r in range(P2 + 1)]
        dpairs = nat.buf(P2 * qh * 64 * 2 * 4)
        widest = max(b2[r + 1] - b2[r] for r in range(P2))
        dsc = nat.buf(qh * widest * 4)
        for r in range(P2):
            n = b2[r + 1] - b2[r]
            assert nat.lib.m40llm_kvcache_score_old_blocks_async(nat.ctx, kv, 0, dq.ptr, qh, L, b2[r], b2[r + 1], dsc.ptr) == 0
            assert nat.lib.m40llm_topk_pairs_async(nat.ctx, dsc.ptr, qh, n, n, b2[r], top, dpairs.ptr + r * qh * 64 * 8) == 0
        dglob, dgsc = nat.buf(qh * 64 * 4), nat.buf(qh * 64 * 4)
        assert nat.lib.m40llm_topk_merge_pairs_async(nat.ctx, dpairs.ptr, P2, qh, top, dglob.ptr, dgsc.ptr) == 0
        dtr = nat.buf(P2 * qh * (2 + hd) * 4)
        for r in range(P2):
            base = dtr.ptr + r * qh * (2 + hd) * 4
            rc = nat.lib.m40llm_attention_compressed_selected_partial_async(
                nat.ctx, kv, 0, dq.ptr, qh, L, dglob.ptr, b2[r], b2[r + 1], 1 if r == P2 - 1 else 0,
                base, base + qh * 4, base + 2 * qh * 4)
            assert rc == 0, rc
        assert nat.lib.m40llm_attention_merge_gathered_async(nat.ctx, dtr.ptr, P2, qh, hd, do.ptr) == 0
        nat.sync(1)
        dev_glob = dglob.download(np.uint32, (qh, 64))
        dev_gsc = dgsc.download(np.float32, (qh, 64))
        for h in range(qh):
            _, _, _, s64 = O.block_select_head(old_k, q[h * hd:(h + 1) * hd], h // (qh // kvh), L - R, bs, top)
            assert_selection_matches([int(b) for b in dev_glob[h, :top]], [int(b) for b in esel[h, :ecnt[h]]], s64,
                                     what=f"device top-k over {P2} ranks, head {h}")
            assert np.all(np.diff(dev_gsc[h, :top]) <= 0), "scores must be in descending order"
        assert_close(do.download(np.float32, q.shape), exp, what=f"device-side split-K over {P2} ranks")
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_topk_pairs_rules(nat):
    """Ties go to the lower block, NaN and scores <= -1e30 are never chosen, short candidate lists leave empty slots,
    and a list shorter than a previous call's leaves nothing stale behind."""
    E = 0xFFFFFFFF
    s = np.array([[1.0, 3.0, 3.0, np.nan, -2e30, 2.0, 3.0], [0.5, 0.5, 0.5, 0.5, 0.5, 0.5, 0.5]], np.float32)
    ds, dp = nat.buf(s), nat.buf(2 * 64 * 2 * 4)
    for top, want0, want1 in ((64, [101, 102, 106, 105, 100], [100, 101, 102, 103, 104, 105, 106]), (2, [101, 102], [100, 101])):
        assert nat.lib.m40llm_topk_pairs_async(nat.ctx, ds.ptr, 2, 7, 7, 100, top, dp.ptr) == 0
        nat.sync(1)
        pairs = dp.download(np.uint32, (2, 64, 2))
        ids = pairs[:, :, 1]
        assert list(ids[0, :len(want0)]) == want0 and (ids[0, len(want0):] == E).all()
        assert list(ids[1, :len(want1)]) == want1 and (ids[1, len(want1):] == E).all()
        sc = pairs[:, :, 0].view(np.float32)
        assert sc[0, 0] == 3.0 and sc[0, 1] == 3.0
    assert nat.lib.m40llm_topk_pairs_async(nat.ctx, ds.ptr, 2, 7, 7, 0, 65, dp.ptr) == -2
    assert nat.lib.m40llm_topk_pairs_async(nat.ctx, ds.ptr, 2, 5000, 5000, 0, 8, dp.ptr) == -2
    assert nat.lib.m40llm_topk_merge_pairs_async(nat.ctx, None, 1, 2, 8, dp.ptr, None) == -1
    nat.free_all()


def test_argument_errors(nat):
    kvd = nat.kv_dense(64, 1, 2, 64)
    kvc = nat.kv_compressed(64, 1, 2, 64, 8, 4, 3)
    q = nat.buf(np.zeros(8 * 64, np.float32))
    f = nat.lib.m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async
    assert f(nat.ctx, kvd, 0, q.ptr, 8, 16, 8, 4, 3, q.ptr) == -16   # no fp16-k/q4-v backing
    assert f(nat.ctx, kvc, 0, None, 8, 16, 8, 4, 3, q.ptr) == -1
    assert f(nat.ctx, kvc, 1, q.ptr, 8, 16, 8, 4, 3, q.ptr) == -2
    assert f(nat.ctx, kvc, 0, q.ptr, 8, 0, 8, 4, 3, q.ptr) == -3
    assert f(nat.ctx, kvc, 0, q.ptr, 8, 65, 8, 4, 3, q.ptr) == -3
    assert f(nat.ctx, kvc, 0, q.ptr, 7, 16, 8, 4, 3, q.ptr) == -4
    assert f(nat.ctx, kvc, 0, q.ptr, 8, 16, 8, 4, 0, q.ptr) == -6
    assert f(nat.ctx, kvc, 0, q.ptr, 8, 16, 8, 4, 65, q.ptr) == -6
    assert f(nat.ctx, kvc, 0, q.ptr, 8, 16, 8, 0, 3, q.ptr) == -6
    g = nat.lib.m40llm_attention_last_token_f32_gqa_block_summary_lossy_async
    assert g(nat.ctx, kvc, 0, q.ptr, 8, 16, 8, 4, 3, q.ptr) == -100
    nat.lib.m40llm_kvcache_destroy(kvd)
    nat.lib.m40llm_kvcache_destroy(kvc)
    nat.free_all()
