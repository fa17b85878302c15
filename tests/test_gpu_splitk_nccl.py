"""Split-K attention of one long sequence over real GPUs: one process per GPU, NCCL all-gather of the block scores
and of the (max, sum, out) triples, compute through the C ABI's partial entry points. Needs two visible GPUs (skipped
otherwise); the rank logic itself is covered on CPU by test_splitk_gloo.py."""
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
        # compressed cache: every rank holds the sequence, reads only its own block range (and the last rank the ring)
        kvc = nat.kv_compressed(L, 1, KVH, HD, R, BS, TOP)
        nat.kv_fill(kvc, 0, k, v, final_len=L)
        legs = splitk.NativeLegs(nat.lib, nat.ctx, kvc, dq, QH, HD, 0, L).legs()
        nb = (L - R + BS - 1) // BS
        out_c, blocks = splitk.compressed_split_k(legs, nb, TOP)
        # dense cache, token-range split
        kvd = nat.kv_dense(L, 1, KVH, HD)
        nat.kv_fill(kvd, 0, k, v)
        legs_d = splitk.NativeLegs(nat.lib, nat.ctx, kvd, dq, QH, HD, 0, L).legs()
        out_d = splitk.dense_split_k(legs_d, L)
        torch.cuda.synchronize()
        if rank == 0:
            np.savez(out_path, out_c=out_c.cpu().numpy(), blocks=blocks, out_d=out_d.cpu().numpy())
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
    world = 2
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as d:
        out_path = os.path.join(d, "out.npz")
        procs = [ctx.Process(target=_rank, args=(r, world, os.path.join(d, "store"), out_path)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0, f"rank exited with {p.exitcode}"
        got = np.load(out_path)
        out_c, blocks, out_d = got["out_c"], got["blocks"], got["out_d"]
    k, v, q = _inputs()
    old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k, v, L, R)
    exp_c, esel, ecnt, _ = O.attention_compressed(old_k, q4, sc, rk, rv, q, QH, L, R, BS, TOP)
    G = QH // KVH
    for h in range(QH):
        s64 = O.block_select_head(old_k, q[h * HD:(h + 1) * HD], h // G, L - R, BS, TOP)[3]
        assert_selection_matches([int(b) for b in blocks[h, :TOP]], [int(b) for b in esel[h, :ecnt[h]]], s64,
                                 what=f"head {h}")
    assert_close(out_c, exp_c, what="compressed split-K over 2 GPUs")
    assert_close(out_d, O.attention_gqa(k, v, q, QH, L), what="dense split-K over 2 GPUs")
