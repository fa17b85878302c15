"""Split-K attention of one long sequence over real GPUs: one process per GPU, every rank holding only its own block
(or token) range, NCCL all-gathers of the local top-k (score, block) pairs and of the (max, sum, out) triples enqueued on
the library's decode stream, selection and merge on the device. Needs two visible GPUs (skipped otherwise; up to four are
used); the rank logic itself is covered on CPU by test_splitk_gloo.py."""
import os
import sys
import tempfile

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

pytestmark = pytest.mark.gpu

QH, KVH, HD, L, R, BS, TOP = 16, 2, 128, 6000, 512, 64, 16


def _inputs():
    rng = np.random.default_rng(41)
    k = rng.standard_normal((L, KVH, HD)).astype(np.float16)
    v = rng.standard_normal((L, KVH, HD)).astype(np.float16)
    q = rng.standard_normal(QH * HD).astype(np.float32)
    return k, v, q


def _rank(rank, world, store, out_path):
    import torch
    import torch.distributed as dist
    import helpers
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{store}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        pkg = helpers.load_package()
        nat = helpers.Native(pkg.native.lib(), device=rank)
        splitk = pkg.splitk
        k, v, q = _inputs()
        dev = torch.device("cuda", rank)
        dq = torch.from_numpy(q).to(dev)
        old_len = L - R
        nb = (old_len + BS - 1) // BS
        # compressed cache: a rank loads ONLY the tokens of its own block range (the last rank also the recent ring);
        # everything else in its cache stays zero and must never be read
        b0, b1 = splitk.block_ranges(nb, world)[rank]
        kvc = nat.kv_compressed(L, 1, KVH, HD, R, BS, TOP)
        t0, t1 = b0 * BS, min(b1 * BS, old_len)
        if rank == world - 1:
            t1 = L
        nat.kv_fill(kvc, 0, k[t0:t1], v[t0:t1], final_len=L, tok_begin=t0)
        sk = splitk.DeviceSplitK(nat.lib, nat.ctx, kvc, dq, QH, HD, 0, L)
        out_c, blocks = sk.compressed(nb, TOP)
        out_c2, _ = sk.compressed(nb, TOP)          # a second call reuses every buffer
        nat.sync(1)
        out_c, out_c2 = out_c.cpu().numpy().copy(), out_c2.cpu().numpy().copy()
        blocks = blocks.cpu().numpy().view(np.uint32).copy()
        # dense cache, token-range split: again only the rank's own tokens are loaded
        kvd = nat.kv_dense(L, 1, KVH, HD)
        d0, d1 = splitk.token_ranges(L, world)[rank]
        nat.kv_fill(kvd, 0, k[d0:d1], v[d0:d1], final_len=L, tok_begin=d0)
        skd = splitk.DeviceSplitK(nat.lib, nat.ctx, kvd, dq, QH, HD, 0, L)
        out_d = skd.dense(L)
        nat.sync(1)
        out_d = out_d.cpu().numpy().copy()
        st = np.zeros(1, np.uint32)
        assert nat.lib.m40llm_context_take_device_status(nat.ctx, st.ctypes.data) == 0 and st[0] == 0
        if rank == 0:
            np.savez(out_path, out_c=out_c, out_c2=out_c2, blocks=blocks, out_d=out_d)
        nat.lib.m40llm_kvcache_destroy(kvc)
        nat.lib.m40llm_kvcache_destroy(kvd)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_split_k_two_gpus(O):
    import torch
    import torch.multiprocessing as mp
    from helpers import assert_close, assert_selection_matches
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as d:
        out_path = os.path.join(d, "out.npz")
        procs = [ctx.Process(target=_rank, args=(r, world, os.path.join(d, "store"), out_path)) for r in range(world)]
        try:
            for p in procs:
                p.start()
            for p in procs:
                p.join(300)
                assert p.exitcode == 0, f"rank exited with {p.exitcode}"
        finally:
            # never leave a rank behind in a collective on a shared GPU
            for p in procs:
                if p.is_alive():
                    p.terminate()
            for p in procs:
                p.join(10)
                if p.is_alive():
                    p.kill()
        got = np.load(out_path)
        out_c, out_c2, blocks, out_d = got["out_c"], got["out_c2"], got["blocks"], got["out_d"]
    k, v, q = _inputs()
    old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k, v, L, R)
    exp_c, esel, ecnt, _ = O.attention_compressed(old_k, q4, sc, rk, rv, q, QH, L, R, BS, TOP)
    G = QH // KVH
    for h in range(QH):
        s64 = O.block_select_head(old_k, q[h * HD:(h + 1) * HD], h // G, L - R, BS, TOP)[3]
        assert_selection_matches([int(b) for b in blocks[h, :TOP]], [int(b) for b in esel[h, :ecnt[h]]], s64,
                                 what=f"head {h}")
    assert_close(out_c, exp_c, what=f"compressed split-K over {world} GPUs")
    assert np.array_equal(out_c, out_c2), "a repeated call must reproduce the result bit for bit"
    assert_close(out_d, O.attention_gqa(k, v, q, QH, L), what=f"dense split-K over {world} GPUs")
    print(f"split-K over {world} GPUs (NCCL all-gather of top-k pairs and of triples): compressed and dense outputs and the "
          f"block lists match the oracle")
