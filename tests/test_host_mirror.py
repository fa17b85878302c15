"""Host-side mirror (C++: kv compression config, decode batch plan) against the reference's own unit tests:
src/kv_compression.rs:326-427 and src/decode_batch.rs:380-411. Pure host logic, runs on CPU."""
import pytest


@pytest.fixture(scope="module")
def H(pkg):
    return pkg.host


def test_default_config_validates_direct_fp16_k_q4_v(H):
    cfg = H.default_kv_cfg()
    assert H.validate(cfg) == ""
    assert H.validate(cfg, 1, 2048, 64) == "" and H.validate(cfg, 1, 2048, 128) == ""
    assert (cfg.mode, cfg.top_blocks, cfg.exact_old_backing, cfg.exact_old_attention) == \
        (H.MODE_BLOCK_SELECT_EXACT, 8, H.BACKING_FP16K_Q4V, H.ATTN_FP16K_Q4V_DIRECT)
    assert (cfg.recent_window, cfg.block_size) == (1024, 32)
    assert H.validate(cfg, 2, 2048, 128) == ""


def test_dense_reference_config_is_explicit(H):
    cfg = H.dense_kv_cfg()
    assert H.validate(cfg) == "" and H.validate(cfg, 1, 16, 128) == "" and H.validate(cfg, 2, 16, 128) == ""


def test_runtime_support_rejections(H):
    cfg = H.default_kv_cfg()
    assert "kv_recent_window" in H.validate(cfg, 1, 512, 64)
    bad = H.default_kv_cfg()
    bad.exact_old_backing, bad.exact_old_attention = H.BACKING_Q8, H.ATTN_Q8_DIRECT
    assert "head_dim=128" in H.validate(bad, 1, 2048, 128)
    assert H.validate(bad, 1, 2048, 64) == ""            # valid for the reference ...
    assert "only" in H.validate(bad, 2, 2048, 64)        # ... but a mode this library does not implement
    big = H.default_kv_cfg()
    big.top_blocks = 65
    assert "limit of 64" in H.validate(big, 1, 2048, 64)


def test_mismatched_backing_and_mode(H):
    cfg = H.default_kv_cfg()
    cfg.exact_old_backing = H.BACKING_DENSE
    assert "requires kv_exact_old_backing=fp16-k-q4-v" in H.validate(cfg)
    off = H.dense_kv_cfg()
    off.exact_old_backing = H.BACKING_Q8
    assert "requires kv_compress_mode" in H.validate(off)
    z = H.default_kv_cfg()
    z.recent_window = 0
    assert "kv_recent_window must be > 0" in H.validate(z)
    z = H.default_kv_cfg()
    z.top_blocks = 0
    assert "top_blocks must be > 0" in H.validate(z)


def test_decode_batch_keeps_active_mixed_lengths(H):
    reqs = [(10, 2, 5, True), (11, 3, 7, False), (12, 4, 1, True), (13, 5, 9, False), (14, 6, 3, True)]
    ids, lens, rids = H.plan_from_requests(reqs)
    assert list(ids) == [2, 4, 6] and list(lens) == [5, 1, 3] and list(rids) == [10, 12, 14]


def test_decode_batch_rejections(H):
    with pytest.raises(ValueError, match="at least one active request"):
        H.plan_from_requests([(1, 0, 1, False)])
    with pytest.raises(ValueError, match="zero kv_len"):
        H.plan_from_requests([(1, 0, 0, True)])
