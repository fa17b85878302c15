"""The allocation-free dense attention entry point (m40llm_attention_last_token_f32_gqa_static_async) through the
C ABI against the regular entry point and the oracle. Collected last on purpose: it must hold both after every other
test has used the device and alone in a fresh process (`pytest tests/test_zz_no_alloc.py -m gpu`)."""
import numpy as np
import pytest

from helpers import assert_close

pytestmark = pytest.mark.gpu

ERR_UNSUPPORTED, ERR_LIMIT = -100, -101


def scratch_generation(nat):
    g = np.zeros(1, np.uint64)
    assert nat.lib.m40llm_context_scratch_generation(nat.ctx, g.ctypes.data) == 0
    return int(g[0])


def both(nat, kv, seq, q, qh, L):
    """(regular entry point, static entry point) outputs for the same call."""
    dq, d_ref, d_new = nat.buf(q), nat.buf(q.nbytes), nat.buf(q.nbytes)
    assert nat.lib.m40llm_attention_last_token_f32_gqa_async(nat.ctx, kv, seq, dq.ptr, qh, L, d_ref.ptr) == 0
    nat.sync(1)
    rc = nat.lib.m40llm_attention_last_token_f32_gqa_static_async(nat.ctx, kv, seq, dq.ptr, qh, L, d_new.ptr)
    assert rc == 0, rc
    nat.sync(1)
    return d_ref.download(np.float32, q.shape), d_new.download(np.float32, q.shape)


@pytest.mark.parametrize("qh,kvh,hd,max_seq", [(32, 8, 128, 8192), (8, 2, 64, 700)])
def test_static_matches_regular_twice_in_a_row(nat, O, qh, kvh, hd, max_seq):
    rng = np.random.default_rng(hd + qh)
    kv = nat.kv_dense(max_seq, 2, kvh, hd)
    k = rng.standard_normal((max_seq, kvh, hd)).astype(np.float16)
    v = rng.standard_normal((max_seq, kvh, hd)).astype(np.float16)
    nat.kv_fill(kv, 1, k, v)
    # two calls back to back share the fixed partials array; lengths cover one split, several splits, a ragged tail
    for L in (max_seq, max_seq - 37, 1, 64, 300, max_seq):
        q = rng.standard_normal(qh * hd).astype(np.float32)
        ref, new = both(nat, kv, 1, q, qh, L)
        assert_close(new, ref, what=f"static vs regular {qh}/{kvh} d{hd} L{L}")
        assert_close(new, O.attention_gqa(k, v, q, qh, L), what=f"static vs oracle {qh}/{kvh} d{hd} L{L}")
    status = np.zeros(1, np.uint32)
    assert nat.lib.m40llm_context_take_device_status(nat.ctx, status.ctypes.data) == 0 and status[0] == 0
    nat.lib.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_static_rejects_what_it_cannot_hold(nat):
    # 64 q heads x 128 splits x (2 + 128) floats = 1 064 960 > 2^20: refused before any launch (a 131072-token sequence
    # is cut into the maximum of 128 splits of 1024 tokens)
    kv = nat.kv_dense(131072, 1, 4, 128)
    q = np.zeros(64 * 128, np.float32)
    dq, do = nat.buf(q), nat.buf(q.nbytes)
    L = nat.lib
    assert L.m40llm_attention_last_token_f32_gqa_static_async(nat.ctx, kv, 0, dq.ptr, 64, 131072, do.ptr) == ERR_LIMIT
    assert L.m40llm_attention_last_token_f32_gqa_static_async(nat.ctx, kv, 0, dq.ptr, 64, 16384, do.ptr) == 0   # fits
    # argument checks are the regular entry point's
    assert L.m40llm_attention_last_token_f32_gqa_static_async(nat.ctx, kv, 1, dq.ptr, 64, 16, do.ptr) == -2
    assert L.m40llm_attention_last_token_f32_gqa_static_async(nat.ctx, kv, 0, dq.ptr, 64, 0, do.ptr) == -3
    assert L.m40llm_attention_last_token_f32_gqa_static_async(nat.ctx, kv, 0, dq.ptr, 6, 16, do.ptr) == -6
    L.m40llm_kvcache_destroy(kv)
    kv = nat.kv_dense(64, 1, 2, 32)  # head_dim outside the tiled kernel's shapes
    assert L.m40llm_attention_last_token_f32_gqa_static_async(nat.ctx, kv, 0, dq.ptr, 4, 16, do.ptr) == ERR_UNSUPPORTED
    L.m40llm_kvcache_destroy(kv)
    nat.free_all()


def test_static_call_allocates_nothing(pkg, O):
    """The property the entry point exists for. On a context of its own, where the regular attention path has never
    run, multi-split static calls leave the context's scratch arenas as they were (the growth counter does not move)
    and, once the kernels' code is resident after a first call, the device's free memory does not change."""
    import helpers
    import torch

    own = helpers.Native(pkg.native.lib())
    try:
        qh, kvh, hd, max_seq = 32, 8, 128, 8192
        rng = np.random.default_rng(99)
        kv = own.kv_dense(max_seq, 1, kvh, hd)
        k = rng.standard_normal((max_seq, kvh, hd)).astype(np.float16)
        v = rng.standard_normal((max_seq, kvh, hd)).astype(np.float16)
        own.kv_fill(kv, 0, k, v)
        q = rng.standard_normal(qh * hd).astype(np.float32)
        dq, do = own.buf(q), own.buf(q.nbytes)
        gen0 = scratch_generation(own)
        f = own.lib.m40llm_attention_last_token_f32_gqa_static_async
        assert f(own.ctx, kv, 0, dq.ptr, qh, max_seq, do.ptr) == 0  # set-up call: symbol lookup, kernel attributes
        own.sync(1)
        free0 = torch.cuda.mem_get_info(0)[0]
        for L in (max_seq, 5000, 129, max_seq):
            assert f(own.ctx, kv, 0, dq.ptr, qh, L, do.ptr) == 0
            own.sync(1)
            assert_close(do.download(np.float32, q.shape), O.attention_gqa(k, v, q, qh, L), what=f"own context L{L}")
        assert torch.cuda.mem_get_info(0)[0] == free0, "device free memory moved across static calls"
        assert scratch_generation(own) == gen0, "a static call grew a scratch arena"
        own.lib.m40llm_kvcache_destroy(kv)
    finally:
        own.free_all()
        own.lib.m40llm_destroy_context(own.ctx)
