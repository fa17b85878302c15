"""Host logic of the multi-GPU paths on CPU: shard plans, the global top-k rule, and the split-K exchange run as two
`gloo` ranks whose compute legs are a numpy restatement, checked against the oracle's single-process answer."""
import os
import sys
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

from helpers import assert_close, assert_selection_matches, load_package  # noqa: E402

splitk = load_package().splitk


# ----------------------------------------------------------------------------- plans
def test_block_ranges_cover_and_balance():
    for n in (0, 1, 7, 8, 9, 504, 505):
        for w in (1, 2, 3, 4, 8):
            r = splitk.block_ranges(n, w)
            assert len(r) == w and r[0][0] == 0 and r[-1][1] == n
            assert all(r[i][1] == r[i + 1][0] for i in range(w - 1))
            sizes = [e - b for b, e in r]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        splitk.block_ranges(4, 0)


def test_token_ranges_are_tile_aligned():
    for L in (1, 63, 64, 65, 1000, 32768, 32769):
        for w in (1, 2, 4, 8):
            r = splitk.token_ranges(L, w)
            assert r[0][0] == 0 and r[-1][1] == L and all(r[i][1] == r[i + 1][0] for i in range(w - 1))
            assert all(b % 64 == 0 for b, e in r if e > b)


def test_shard_sequences_balances_contexts():
    rng = np.random.default_rng(4)
    lens = rng.integers(128, 16385, size=256)
    for w in (1, 2, 4, 8):
        shards = splitk.shard_sequences(lens, w)
        assert sorted(i for s in shards for i in s) == list(range(256))
        loads = [int(lens[s].sum()) for s in shards]
        assert max(loads) - min(loads) <= int(lens.max())      # longest-first greedy bound
        assert max(loads) <= 1.02 * sum(loads) / w
    assert splitk.shard_sequences([5, 5, 5], 2) == [[0, 2], [1]]
    # equal row counts per rank (the weak-scaling deal: 32 sequences each) still balance the tokens
    for w in (2, 4, 8):
        lens = rng.integers(512, 8193, size=32 * w)
        shards = splitk.shard_sequences(lens, w, max_per_rank=32)
        assert all(len(s) == 32 for s in shards) and sorted(i for s in shards for i in s) == list(range(32 * w))
        loads = [int(lens[s].sum()) for s in shards]
        assert max(loads) <= 1.01 * sum(loads) / w
    with pytest.raises(ValueError):
        splitk.shard_sequences([1, 2, 3], 2, max_per_rank=1)
    assert splitk.shard_sequences([], 2) == [[], []]


def test_select_global_topk_rule():
    E = splitk.EMPTY_BLOCK
    s = np.array([[1.0, 3.0, 3.0, np.nan, -2e30, 2.0, 3.0]], np.float32)
    got = splitk.select_global_topk(s, 4)
    assert got.shape == (1, 64) and list(got[0, :5]) == [1, 2, 6, 5, E]          # ties -> lower index
    got = splitk.select_global_topk(s, 64)
    assert list(got[0, :6]) == [1, 2, 6, 5, 0, E]                                  # NaN and <= -1e30 never chosen
    assert (splitk.select_global_topk(np.zeros((3, 0), np.float32), 8) == E).all()
    with pytest.raises(ValueError):
        splitk.select_global_topk(s, 65)


def test_pair_exchange_equals_global_selection():
    """Local top-k pairs per block range, then the merge of the gathered pairs, give the list the global rule gives
    on the whole score matrix: every world size, ties across ranges, ranges shorter than the top count."""
    rng = np.random.default_rng(12)
    E = splitk.EMPTY_BLOCK
    for nb, top in ((504, 64), (37, 8), (5, 8), (64, 64), (130, 1)):
        scores = rng.standard_normal((6, nb)).astype(np.float32)
        scores[0, ::7] = scores[0, 3]            # ties that straddle rank boundaries
        scores[1, 5:9] = np.nan
        scores[2, :] = -2e30                     # nothing selectable
        want = splitk.select_global_topk(scores, top)
        for world in (1, 2, 3, 8):
            parts = [splitk.host_topk_pairs(scores[:, b:e], b, top) for b, e in splitk.block_ranges(nb, world)]
            got = splitk.host_merge_pairs(np.stack(parts), top)
            assert np.array_equal(got, want), (nb, top, world)
    assert (splitk.host_merge_pairs(np.stack([splitk.host_topk_pairs(np.zeros((2, 0), np.float32), 0, 4)]), 4) == E).all()


def test_select_global_topk_matches_oracle_selection():
    O = __import__("oracle.oracle", fromlist=["oracle"])
    rng = np.random.default_rng(8)
    kvh, hd, old_len, bs, top = 2, 64, 1000, 16, 12
    old_k = rng.standard_normal((old_len, kvh, hd)).astype(np.float16)
    for h in range(4):
        q = rng.standard_normal(hd).astype(np.float32)
        blocks, _, s32, s64 = O.block_select_head(old_k, q, h // 2, old_len, bs, top)
        mine = splitk.select_global_topk(s32[None, :], top)[0]
        assert_selection_matches([int(b) for b in mine[:top]], [int(b) for b in blocks], s64, what=f"head {h}")


def test_merge_triples_matches_oracle_merge():
    O = __import__("oracle.oracle", fromlist=["oracle"])
    rng = np.random.default_rng(5)
    parts, heads, hd = 5, 6, 32
    m = rng.standard_normal((parts, heads)).astype(np.float32) * 4
    l = rng.uniform(0.5, 50, (parts, heads)).astype(np.float32)
    o = rng.standard_normal((parts, heads, hd)).astype(np.float32) * l[:, :, None]
    assert_close(splitk.merge_triples(m, l, o), O.merge_partials(m, l, o), what="merge")
    # one part alone is its own normalisation; empty parts (l == 0) are ignored
    l2, m2 = l.copy(), m.copy()
    l2[1:] = 0
    m2[1:] = -np.inf
    assert_close(splitk.merge_triples(m2, l2, o), (o[0] / l[0][:, None]).reshape(-1), what="single live part")


# ----------------------------------------------------------------------------- two gloo ranks
QH, KVH, HD, L, R, BS, TOP = 8, 2, 64, 1500, 100, 16, 8


def _state():
    O = __import__("oracle.oracle", fromlist=["oracle"])
    rng = np.random.default_rng(77)
    k = rng.standard_normal((L, KVH, HD)).astype(np.float16)
    v = rng.standard_normal((L, KVH, HD)).astype(np.float16)
    q = rng.standard_normal(QH * HD).astype(np.float32)
    return O, k, v, q


def _partial(q, keys, vals):
    """Unnormalised (m, l, o) of one head over the given f32 keys/values (numpy restatement of a leg)."""
    if keys.shape[0] == 0:
        return np.float32(-np.inf), np.float32(0), np.zeros(HD, np.float32)
    logit = (keys @ q).astype(np.float32) * np.float32(1.0 / np.sqrt(HD))
    m = logit.max()
    p = np.exp(logit - m).astype(np.float32)
    return m, p.sum(dtype=np.float32), (p[:, None] * vals).sum(axis=0).astype(np.float32)


def _worker(rank, world, store_path, results):
    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
    try:
        O, k, v, q = _state()
        G = QH // KVH
        old_len = L - R
        nb = (old_len + BS - 1) // BS
        old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k, v, L, R)
        vq = O.q4_dequant(q4, sc)                                  # f32 [old_len, kvh, hd]
        kf = old_k.astype(np.float32)

        def score(b0, b1):
            rows = [O.block_select_head(old_k, q[h * HD:(h + 1) * HD], h // G, old_len, BS, TOP)[2][b0:b1]
                    for h in range(QH)]
            return torch.from_numpy(np.stack(rows).astype(np.float32))

        def pack(m, l, o):  # one message per rank: m | l | o
            return torch.from_numpy(np.concatenate([m, l, o.reshape(-1)]).astype(np.float32))

        def topk_pairs(scores, b0, top):
            return torch.from_numpy(splitk.host_topk_pairs(scores.numpy(), b0, top))

        def merge_pairs(pairs, top):
            return splitk.host_merge_pairs(pairs.numpy(), top)

        def attend_blocks(blocks, b0, b1, include_recent):
            m, l, o = np.empty(QH, np.float32), np.empty(QH, np.float32), np.empty((QH, HD), np.float32)
            for h in range(QH):
                toks = [t for b in blocks[h] if b != splitk.EMPTY_BLOCK and b0 <= b < b1
                        for t in range(int(b) * BS, min((int(b) + 1) * BS, old_len))]
                keys, vals = kf[toks, h // G], vq[toks, h // G]
                if include_recent:
                    slots = [t % R for t in range(old_len, L)]
                    keys = np.concatenate([keys, rk[slots, h // G].astype(np.float32)])
                    vals = np.concatenate([vals, rv[slots, h // G].astype(np.float32)])
                m[h], l[h], o[h] = _partial(q[h * HD:(h + 1) * HD], keys, vals)
            return pack(m, l, o)

        def attend_tokens(t0, t1):
            m, l, o = np.empty(QH, np.float32), np.empty(QH, np.float32), np.empty((QH, HD), np.float32)
            for h in range(QH):
                m[h], l[h], o[h] = _partial(q[h * HD:(h + 1) * HD], k[t0:t1, h // G].astype(np.float32),
                                            v[t0:t1, h // G].astype(np.float32))
            return pack(m, l, o)

        def merge(triples):
            t = triples.numpy()
            return torch.from_numpy(splitk.merge_triples(t[:, :QH], t[:, QH:2 * QH], t[:, 2 * QH:].reshape(-1, QH, HD)))

        legs = splitk.Legs(score, topk_pairs, merge_pairs, attend_blocks, attend_tokens, merge)
        out_c, blocks = splitk.compressed_split_k(legs, nb, TOP)
        out_d = splitk.dense_split_k(legs, L)
        results[rank] = (out_c.numpy().copy(), blocks.copy(), out_d.numpy().copy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_split_k_exchange_over_gloo(world):
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as d, ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, os.path.join(d, "store"), results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0, f"rank exited with {p.exitcode}"
        got = [results[r] for r in range(world)]
    O, k, v, q = _state()
    old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k, v, L, R)
    exp_c, esel, ecnt, _ = O.attention_compressed(old_k, q4, sc, rk, rv, q, QH, L, R, BS, TOP)
    exp_d = O.attention_gqa(k, v, q, QH, L)
    G = QH // KVH
    for r in range(world):
        out_c, blocks, out_d = got[r]
        assert np.array_equal(blocks, got[0][1]), "ranks disagree on the global block list"
        for h in range(QH):
            s64 = O.block_select_head(old_k, q[h * HD:(h + 1) * HD], h // G, L - R, BS, TOP)[3]
            assert_selection_matches([int(b) for b in blocks[h, :TOP]], [int(b) for b in esel[h, :ecnt[h]]], s64,
                                     what=f"rank {r} head {h}")
        assert_close(out_c, exp_c, what=f"compressed split-K, rank {r} of {world}")
        assert_close(out_d, exp_d, what=f"dense split-K, rank {r} of {world}")
