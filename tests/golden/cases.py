"""Seeded input definitions shared by the golden-vector generator (make_golden.py) and the tests that
consume the vectors. Inputs are regenerated from the seed on both sides, so only outputs are stored."""
from __future__ import annotations

import numpy as np


def rng_for(name: str) -> np.random.Generator:
    return np.random.default_rng(abs(hash_name(name)) % (2 ** 32))


def hash_name(name: str) -> int:
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


NORM_CASES = {"norm_2x8": (2, 8), "norm_3x2048": (3, 2048), "norm_1x4096": (1, 4096)}
ROPE_CASES = {  # name: (rows, heads, hd, past_len, base, layout)
    "rope_adj_small": (1, 2, 4, 3, 1e4, 0), "rope_adj_64": (2, 8, 64, 2047, 1e4, 0),
    "rope_adj_128": (1, 8, 128, 8191, 5e5, 0), "rope_neox_128": (2, 4, 128, 32767, 1e6, 1),
    "rope_neox_64": (1, 4, 64, 100, 1e4, 1),
}
GEMM_CASES = {"gemm_3x17x64": (3, 17, 64), "gemm_1x256x512": (1, 256, 512), "gemm_2x96x1000": (2, 96, 1000)}
ATTN_CASES = {  # name: (q_heads, kv_heads, hd, L)
    "attn_toy": (8, 2, 64, 256), "attn_tiny": (32, 4, 64, 512), "attn_hd128": (16, 2, 128, 300),
    "attn_hd32": (4, 1, 32, 40), "attn_hd128_long": (8, 2, 128, 2048),
}
BATCH_CASES = {"batched_hd64": (4, 2, 64, [1, 3, 5, 200])}
Q4_CASES = {  # name: (q_heads, kv_heads, hd, L, R, bs, top)
    "q4_all_selected": (4, 2, 64, 16, 4, 4, 3), "q4_partial_block": (4, 2, 128, 5, 4, 32, 8),
    "q4_subset_hd64": (8, 2, 64, 600, 64, 16, 5), "q4_subset_hd128": (8, 2, 128, 500, 32, 8, 6),
    "q4_ring_wrap": (8, 2, 64, 45, 8, 4, 3),
}


def norm_inputs(name):
    rows, dim = NORM_CASES[name]
    r = rng_for(name)
    return (r.standard_normal((rows, dim)) * 1.5).astype(np.float32), (1 + 0.2 * r.standard_normal(dim)).astype(np.float32)


def rope_inputs(name):
    rows, heads, hd, *_ = ROPE_CASES[name]
    return rng_for(name).standard_normal((rows, heads * hd)).astype(np.float32)


def gemm_inputs(name):
    M, N, K = GEMM_CASES[name]
    r = rng_for(name)
    a = r.standard_normal((M, K)).astype(np.float32)
    w = (r.standard_normal((N, K)) * 0.05).astype(np.float16)  # GGUF [N][K]; row-major B is w.T
    return a, w


def attn_inputs(name):
    qh, kvh, hd, L = ATTN_CASES[name]
    r = rng_for(name)
    k = r.standard_normal((L, kvh * hd)).astype(np.float32)
    v = r.standard_normal((L, kvh * hd)).astype(np.float32)
    q = r.standard_normal(qh * hd).astype(np.float32)
    return k, v, q


def batch_inputs(name):
    qh, kvh, hd, lens = BATCH_CASES[name]
    r = rng_for(name)
    ks = [r.standard_normal((n, kvh * hd)).astype(np.float32) for n in lens]
    vs = [r.standard_normal((n, kvh * hd)).astype(np.float32) for n in lens]
    q = r.standard_normal((len(lens), qh, hd)).astype(np.float32)
    return ks, vs, q


def q4_inputs(name):
    qh, kvh, hd, L, R, bs, top = Q4_CASES[name]
    r = rng_for(name)
    k = r.standard_normal((L, kvh * hd)).astype(np.float32)
    v = r.standard_normal((L, kvh * hd)).astype(np.float32)
    q = r.standard_normal(qh * hd).astype(np.float32)
    return k, v, q

PREFILL_CASES = {  # name: (q_heads, kv_heads, hd, [(q_len, kv_len), ...])
    "prefill_ref_hd64": (4, 2, 64, [(3, 3), (2, 5), (1, 4)]), "prefill_ref_hd128": (4, 2, 128, [(3, 3), (2, 5), (1, 4)]),
    "prefill_tiles_hd64": (8, 2, 64, [(65, 65), (17, 200)]), "prefill_tiles_hd128": (8, 4, 128, [(130, 130), (1, 70)]),
}


def prefill_inputs(name):
    """(q, k, v, q_offsets, kv_offsets, q_lens, kv_lens): packed f32 rows [tokens][heads][hd]."""
    qh, kvh, hd, pairs = PREFILL_CASES[name]
    rng = rng_for(name)
    ql = np.array([p[0] for p in pairs], np.uint32)
    kl = np.array([p[1] for p in pairs], np.uint32)
    qo = np.concatenate([[0], np.cumsum(ql)[:-1]]).astype(np.uint32)
    ko = np.concatenate([[0], np.cumsum(kl)[:-1]]).astype(np.uint32)
    q = rng.standard_normal((int(ql.sum()), qh, hd)).astype(np.float32)
    k = rng.standard_normal((int(kl.sum()), kvh, hd)).astype(np.float32)
    v = rng.standard_normal((int(kl.sum()), kvh, hd)).astype(np.float32)
    return q, k, v, qo, ko, ql, kl


def prefill_sample_rows(name):
    """Packed q rows whose outputs are stored in the fixture: per sequence the first two, the middle and the last row and
    the rows around the 64-row tile boundary."""
    _, _, _, pairs = PREFILL_CASES[name]
    rows, off = [], 0
    for ql, _ in pairs:
        rows += [off + r for r in sorted({0, 1, ql // 2, ql - 1, 63, 64, 65} & set(range(ql)))]
        off += ql
    return np.array(rows, np.int64)


def cache_sample_tokens(L):
    """Token positions whose cache rows are stored in the fixture (the whole cache would be megabytes)."""
    return sorted(set([0, 1, 2, L // 2, L - 1]) & set(range(L)))
