"""ctypes binding of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and
by the CPU-baseline leg of ``bench.py``. The product library never loads it.

All arrays are numpy, C-contiguous. f16 data travels as ``np.float16`` arrays and
is reinterpreted as ``uint16`` at the boundary.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile next to this file."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


class LayerCfg(C.Structure):
    _fields_ = [
        ("hidden", C.c_uint32), ("q_heads", C.c_uint32), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
        ("ffn", C.c_uint32), ("ffn_q80", C.c_uint32), ("rope_layout", C.c_uint32),
        ("eps", C.c_float), ("rope_base", C.c_float), ("rope_scale", C.c_float),
    ]


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_q4_quantize_head.restype = C.c_float
        _lib.orc_q4_dequant.restype = C.c_float
        _lib.orc_q4_dequant.argtypes = [C.c_uint8, C.c_uint32, C.c_float]
        _lib.orc_block_select_head.restype = C.c_uint32
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _f16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def _u8(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8
    return a


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def f32_to_f16(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.float16)
    lib().orc_f32_to_f16_array(_p(x), _p(out), C.c_size_t(x.size))
    return out


def f16_to_f32(x) -> np.ndarray:
    x = _f16(x)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_f16_to_f32_array(_p(x), _p(out), C.c_size_t(x.size))
    return out


def rms_norm(x, w, eps: float) -> np.ndarray:
    x = _f32(x)
    rows, dim = (1, x.shape[0]) if x.ndim == 1 else x.shape
    w = None if w is None else _f32(w)
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x), _p(w), _p(out), C.c_size_t(rows), C.c_size_t(dim), C.c_float(eps))
    return out


def rope(x, heads: int, head_dim: int, past_len: int, base: float, scale: float, layout: int) -> np.ndarray:
    x = _f32(x).copy()
    rows = x.size // (heads * head_dim)
    lib().orc_rope(_p(x), C.c_size_t(rows), C.c_size_t(heads), C.c_size_t(head_dim), C.c_uint32(past_len),
                   C.c_float(base), C.c_float(scale), C.c_uint32(layout))
    return x


def gemm_f32xf16_gguf(a, w) -> np.ndarray:
    a = _f32(a)
    w = _f16(w)
    a2 = a.reshape(-1, a.shape[-1])
    m, k = a2.shape
    n = w.shape[0]
    assert w.shape[1] == k
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_gemm_f32xf16_gguf(_p(a2), _p(w), _p(out), C.c_int(m), C.c_int(n), C.c_int(k))
    return out.reshape(a.shape[:-1] + (n,))


def gemm_f16xf16_rowmajor(a, b) -> np.ndarray:
    a = _f16(a)
    b = _f16(b)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_gemm_f16xf16_rowmajor(_p(a), _p(b), _p(out), C.c_int(m), C.c_int(n), C.c_int(k))
    return out


def gemm_f32xf16_rowmajor(a, b) -> np.ndarray:
    a = _f32(a)
    b = _f16(b)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_gemm_f32xf16_rowmajor(_p(a), _p(b), _p(out), C.c_int(m), C.c_int(n), C.c_int(k))
    return out


def gemm_f16_storage(a, b) -> np.ndarray:
    a = _f16(a)
    b = _f16(b)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), dtype=np.float16)
    lib().orc_gemm_f16_storage(_p(a), _p(b), _p(out), C.c_int(m), C.c_int(n), C.c_int(k))
    return out


def q80_quantize(w) -> np.ndarray:
    """f32 [..., K] (K % 32 == 0) -> uint8 [..., K/32*34] Q8_0 rows."""
    w = _f32(w)
    k = w.shape[-1]
    assert k % 32 == 0
    out = np.empty(w.shape[:-1] + (k // 32 * 34,), dtype=np.uint8)
    lib().orc_q80_quantize(_p(w), _p(out), C.c_size_t(w.size))
    return out


def q80_to_f32(q, n: int) -> np.ndarray:
    q = _u8(q)
    out = np.empty(n, dtype=np.float32)
    lib().orc_q80_to_f32(_p(q), _p(out), C.c_size_t(n))
    return out


def gemm_f32xq80_gguf(a, wq, n: int) -> np.ndarray:
    a = _f32(a)
    wq = _u8(wq)
    a2 = a.reshape(-1, a.shape[-1])
    m, k = a2.shape
    assert wq.size == n * (k // 32) * 34
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_gemm_f32xq80_gguf(_p(a2), _p(wq), _p(out), C.c_int(m), C.c_int(n), C.c_int(k))
    return out.reshape(a.shape[:-1] + (n,))


def swiglu(g, u) -> np.ndarray:
    g = _f32(g)
    u = _f32(u)
    out = np.empty_like(g)
    lib().orc_swiglu(_p(g), _p(u), _p(out), C.c_size_t(g.size))
    return out


def attention_gqa(k, v, q, q_heads: int, seq_len: int) -> np.ndarray:
    """k, v: f16 [>=seq_len, kv_heads, hd]; q: f32 [q_heads*hd]."""
    k = _f16(k)
    v = _f16(v)
    q = _f32(q)
    kv_heads, hd = k.shape[1], k.shape[2]
    out = np.empty(q_heads * hd, dtype=np.float32)
    rc = lib().orc_attention_gqa(_p(k), _p(v), _p(q), _p(out), C.c_uint32(q_heads), C.c_uint32(kv_heads),
                                 C.c_uint32(hd), C.c_uint32(seq_len))
    assert rc == 0, rc
    return out


def attention_gqa_batched(k, v, seq_ids, seq_lens, q, q_heads: int) -> np.ndarray:
    """k, v: f16 [slots, max_seq, kv_heads, hd]; q: f32 [batch, q_heads, hd]."""
    k = _f16(k)
    v = _f16(v)
    q = _f32(q)
    seq_ids = np.ascontiguousarray(seq_ids, dtype=np.uint32)
    seq_lens = np.ascontiguousarray(seq_lens, dtype=np.uint32)
    _, max_seq, kv_heads, hd = k.shape
    out = np.empty_like(q)
    rc = lib().orc_attention_gqa_batched(_p(k), _p(v), _p(seq_ids), _p(seq_lens), C.c_uint32(len(seq_ids)),
                                         _p(q), _p(out), C.c_uint32(q_heads), C.c_uint32(kv_heads),
                                         C.c_uint32(hd), C.c_uint32(max_seq))
    assert rc == 0, rc
    return out


def q4_quantize(v) -> tuple[np.ndarray, np.ndarray]:
    """v: f16 [tokens, kv_heads, hd] -> (packed u8 [tokens, kv_heads, hd/2], scale f32 [tokens, kv_heads])."""
    v = _f16(v)
    t, h, hd = v.shape
    packed = np.empty((t, h, hd // 2), dtype=np.uint8)
    scale = np.empty((t, h), dtype=np.float32)
    L = lib()
    for i in range(t):
        for j in range(h):
            scale[i, j] = L.orc_q4_quantize_head(_p(v[i, j]), _p(packed[i, j]), C.c_uint32(hd))
    return packed, scale


def q4_dequant(packed, scale) -> np.ndarray:
    """Inverse view used by tests: f32 [tokens, kv_heads, hd] of f16(nibble*scale)."""
    packed = _u8(packed)
    lo = (packed & 0x0F).astype(np.int32)
    hi = (packed >> 4).astype(np.int32)
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = np.where(hi >= 8, hi - 16, hi)
    vals = np.stack([lo, hi], axis=-1).reshape(packed.shape[:-1] + (packed.shape[-1] * 2,)).astype(np.float32)
    vals = vals * _f32(scale)[..., None]
    return f16_to_f32(f32_to_f16(vals))


def block_select_head(old_k, qh, kvh: int, old_len: int, block_size: int, top_blocks: int):
    """Returns (blocks[descending score], their f32 scores, all f32 scores, all f64 scores)."""
    old_k = _f16(old_k)
    qh = _f32(qh)
    kv_heads, hd = old_k.shape[1], old_k.shape[2]
    nb = 0 if old_len == 0 else (old_len + block_size - 1) // block_size
    blocks = np.empty(64, dtype=np.uint32)
    bscores = np.empty(64, dtype=np.float32)
    s32 = np.empty(max(nb, 1), dtype=np.float32)
    s64 = np.empty(max(nb, 1), dtype=np.float64)
    cnt = lib().orc_block_select_head(_p(old_k), _p(qh), C.c_uint32(kvh), C.c_uint32(kv_heads), C.c_uint32(hd),
                                      C.c_uint32(old_len), C.c_uint32(block_size), C.c_uint32(top_blocks),
                                      _p(blocks), _p(bscores), _p(s32), _p(s64))
    return blocks[:cnt].copy(), bscores[:cnt].copy(), s32[:nb].copy(), s64[:nb].copy()


def attention_compressed(old_k, q4_v, q4_scale, recent_k, recent_v, q, q_heads: int, seq_len: int,
                         recent_window: int, block_size: int, top_blocks: int):
    """Returns (out f32 [q_heads*hd], selected [q_heads, 64] u32, counts [q_heads], union_tokens)."""
    old_k = _f16(old_k)
    q4_v = _u8(q4_v)
    q4_scale = _f32(q4_scale)
    recent_k = _f16(recent_k)
    recent_v = _f16(recent_v)
    q = _f32(q)
    kv_heads, hd = recent_k.shape[1], recent_k.shape[2]
    out = np.empty(q_heads * hd, dtype=np.float32)
    sel = np.empty((q_heads, 64), dtype=np.uint32)
    cnt = np.empty(q_heads, dtype=np.uint32)
    union = C.c_uint64(0)
    rc = lib().orc_attention_compressed(_p(old_k), _p(q4_v), _p(q4_scale), _p(recent_k), _p(recent_v), _p(q),
                                        _p(out), C.c_uint32(q_heads), C.c_uint32(kv_heads), C.c_uint32(hd),
                                        C.c_uint32(seq_len), C.c_uint32(recent_window), C.c_uint32(block_size),
                                        C.c_uint32(top_blocks), _p(sel), _p(cnt), C.byref(union))
    assert rc == 0, rc
    return out, sel, cnt, int(union.value)


def attention_block_select_dense(k, v, q, q_heads: int, seq_len: int, recent_window: int, block_size: int,
                                 top_blocks: int) -> np.ndarray:
    k = _f16(k)
    v = _f16(v)
    q = _f32(q)
    kv_heads, hd = k.shape[1], k.shape[2]
    out = np.empty(q_heads * hd, dtype=np.float32)
    rc = lib().orc_attention_block_select_dense(_p(k), _p(v), _p(q), _p(out), C.c_uint32(q_heads),
                                                C.c_uint32(kv_heads), C.c_uint32(hd), C.c_uint32(seq_len),
                                                C.c_uint32(recent_window), C.c_uint32(block_size),
                                                C.c_uint32(top_blocks))
    assert rc == 0, rc
    return out


def merge_partials(m, l, o) -> np.ndarray:
    """m, l: f32 [parts, heads]; o: f32 [parts, heads, hd] -> f32 [heads*hd]."""
    m = _f32(m)
    l = _f32(l)
    o = _f32(o)
    parts, heads, hd = o.shape
    out = np.empty(heads * hd, dtype=np.float32)
    lib().orc_merge_partials(_p(m), _p(l), _p(o), _p(out), C.c_uint32(parts), C.c_uint32(heads), C.c_uint32(hd))
    return out


def compressed_state_from_dense(k, v, seq_len: int, recent_window: int):
    """Host model of the compressed cache after appending tokens 0..seq_len-1 in order
    (cuda/kernels.cu:6108-6250): tokens older than the recent window live as f16 old K and
    q4 old V (quantised from the f16 value that sat in the ring), the newest
    min(seq_len, R) tokens sit in the ring at slot t % R.

    k, v: f16 [>=seq_len, kv_heads, hd] (K already rotated). Returns
    (old_k f16 [old_len,...], q4_v, q4_scale, recent_k f16 [R,...], recent_v)."""
    k = _f16(k)
    v = _f16(v)
    kv_heads, hd = k.shape[1], k.shape[2]
    old_len = max(seq_len - recent_window, 0)
    old_k = np.ascontiguousarray(k[:old_len]) if old_len else np.zeros((0, kv_heads, hd), np.float16)
    if old_len:
        q4_v, q4_scale = q4_quantize(v[:old_len])
    else:
        q4_v = np.zeros((0, kv_heads, hd // 2), np.uint8)
        q4_scale = np.zeros((0, kv_heads), np.float32)
    recent_k = np.zeros((recent_window, kv_heads, hd), np.float16)
    recent_v = np.zeros((recent_window, kv_heads, hd), np.float16)
    for t in range(old_len, seq_len):
        recent_k[t % recent_window] = k[t]
        recent_v[t % recent_window] = v[t]
    return old_k, q4_v, q4_scale, recent_k, recent_v


def decode_layer(cfg: LayerCfg, x, w, K, V, pos: int):
    """One decode layer for one sequence. ``w`` is a dict with keys attn_norm, wq, wk, wv, wo,
    bq, bk, bv (optional), ffn_norm, wg, wu, wd. K, V: f16 [max_seq, kv_heads, hd], updated in place.
    Returns (out [hidden], q_rot [q_heads*hd], att [q_heads*hd])."""
    x = _f32(x)
    out = np.empty(cfg.hidden, dtype=np.float32)
    qd = cfg.q_heads * cfg.head_dim
    dbg_q = np.empty(qd, dtype=np.float32)
    dbg_att = np.empty(qd, dtype=np.float32)
    assert K.flags.c_contiguous and V.flags.c_contiguous and K.dtype == np.float16
    g = lambda name: w.get(name)
    rc = lib().orc_decode_layer(C.byref(cfg), _p(x), _p(out), _p(_f32(w["attn_norm"])), _p(w["wq"]), _p(w["wk"]),
                                _p(w["wv"]), _p(w["wo"]), _p(g("bq")), _p(g("bk")), _p(g("bv")),
                                _p(_f32(w["ffn_norm"])), _p(w["wg"]), _p(w["wu"]), _p(w["wd"]), _p(K), _p(V),
                                C.c_uint32(pos), _p(dbg_q), _p(dbg_att))
    assert rc == 0, rc
    return out, dbg_q, dbg_att


def attention_prefill_varlen(q, k, v, q_offsets, kv_offsets, q_lens, kv_lens, q_heads: int, kv_heads: int, hd: int) -> np.ndarray:
    """Packed causal prefill attention (cuda/kernels.cu:3749-3835): q [total_q, q_heads, hd], k / v [total_kv, kv_heads,
    hd] f32; q row i of a sequence attends its kv rows 0 .. kv_len - q_len + i."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    qo, ko = np.ascontiguousarray(q_offsets, np.uint32), np.ascontiguousarray(kv_offsets, np.uint32)
    ql, kl = np.ascontiguousarray(q_lens, np.uint32), np.ascontiguousarray(kv_lens, np.uint32)
    out = np.zeros_like(q)
    rc = lib().orc_attention_prefill_varlen(_p(q), _p(k), _p(v), _p(qo), _p(ko), _p(ql), _p(kl), C.c_uint32(len(ql)),
                                            C.c_uint32(q_heads), C.c_uint32(kv_heads), C.c_uint32(hd), _p(out))
    assert rc == 0, rc
    return out

