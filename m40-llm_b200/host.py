"""ctypes view of libm40llm_host.so: the C++ host mirror of the reference's decode-layer driver
(src/infer/forward.rs, src/decode_batch.rs, src/kv_compression.rs), which itself calls only the m40llm C ABI."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libm40llm_host.so")

MODE_OFF, MODE_BLOCK_SELECT_EXACT = 0, 5
BACKING_DENSE, BACKING_Q8, BACKING_FP16K_Q4V = 0, 1, 2
ATTN_STAGED, ATTN_Q8_DIRECT, ATTN_FP16K_Q4V_DIRECT = 0, 1, 2


class LayerCfg(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("q_heads", C.c_uint32), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("ffn", C.c_uint32), ("rope_layout", C.c_uint32), ("rms_eps", C.c_float), ("rope_base", C.c_float),
                ("rope_scale", C.c_float)]


class Weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm", "ffn_norm", "wq", "wk", "wv", "wo", "bq", "bk", "bv", "wg", "wu",
                                          "wd")] + [("ffn_q80", C.c_uint32)]


class ModelHead(C.Structure):
    _fields_ = [("embeddings", C.c_void_p), ("output_norm", C.c_void_p), ("lm_head", C.c_void_p), ("vocab", C.c_uint32)]


class KvCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("mode", "recent_window", "block_size", "top_blocks", "representatives",
                                          "representative_policy", "exact_old_backing", "exact_old_attention")]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python m40-llm_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        L.m40host_last_error.restype = C.c_char_p
        L.m40host_kv_cfg_validate.argtypes = [C.POINTER(KvCfg), C.c_uint32, C.c_uint32, C.c_uint32]
        L.m40host_layer_create.restype = C.c_void_p
        L.m40host_layer_create.argtypes = [C.c_void_p, C.POINTER(LayerCfg), C.c_uint32]
        L.m40host_layer_destroy.argtypes = [C.c_void_p]
        L.m40host_layer_forward_host.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(Weights), C.POINTER(KvCfg), C.c_uint32] + \
            [C.c_void_p] * 6 + [C.c_uint32]
        L.m40host_layer_forward_host_begin.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.POINTER(Weights),
                                                       C.POINTER(KvCfg), C.c_uint32] + [C.c_void_p] * 5 + [C.c_uint32]
        L.m40host_layer_forward_host_end.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
        L.m40host_layer_graph_replays.restype = C.c_uint64
        L.m40host_layer_graph_replays.argtypes = [C.c_void_p]
        L.m40host_plan_from_requests.argtypes = [C.c_uint32] + [C.c_void_p] * 8
        L.m40host_model_create.restype = C.c_void_p
        L.m40host_model_create.argtypes = [C.c_void_p, C.POINTER(LayerCfg), C.c_uint32, C.POINTER(Weights),
                                           C.POINTER(ModelHead), C.c_void_p, C.c_uint32]
        L.m40host_model_destroy.argtypes = [C.c_void_p]
        L.m40host_model_begin.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.m40host_model_generate.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
        L.m40host_model_graph_replays.restype = C.c_uint64
        L.m40host_model_graph_replays.argtypes = [C.c_void_p]
        L.m40host_model_launches_per_step.restype = C.c_uint64
        L.m40host_model_launches_per_step.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def last_error() -> str:
    return lib().m40host_last_error().decode()


def default_kv_cfg() -> KvCfg:
    c = KvCfg()
    lib().m40host_kv_cfg_default(C.byref(c))
    return c


def dense_kv_cfg() -> KvCfg:
    """KvCompressionConfig::dense_reference() (src/kv_compression.rs:100-111)."""
    return KvCfg(MODE_OFF, 1024, 32, 8, 0, 0, BACKING_DENSE, ATTN_STAGED)


def validate(cfg: KvCfg, which: int = 0, max_seq_len: int = 0, head_dim: int = 0) -> str:
    rc = lib().m40host_kv_cfg_validate(C.byref(cfg), which, max_seq_len, head_dim)
    return "" if rc == 0 else last_error()


def plan_from_requests(requests):
    """requests: list of (request_id, sequence_id, kv_len, active). Returns (seq_ids, seq_lens, request_ids)."""
    n = len(requests)
    rid = np.array([r[0] for r in requests], np.uint64)
    sid = np.array([r[1] for r in requests], np.uint32)
    kvl = np.array([r[2] for r in requests], np.uint32)
    act = np.array([1 if r[3] else 0 for r in requests], np.uint32)
    ob = C.c_uint32()
    os_, ol, orq = np.zeros(n, np.uint32), np.zeros(n, np.uint32), np.zeros(n, np.uint64)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    rc = lib().m40host_plan_from_requests(n, p(rid), p(sid), p(kvl), p(act), C.cast(C.byref(ob), C.c_void_p), p(os_), p(ol), p(orq))
    if rc != 0:
        raise ValueError(last_error())
    b = ob.value
    return os_[:b].copy(), ol[:b].copy(), orq[:b].copy()


class DecodeLayer:
    """One decode layer step with host buffers in and out (the end-to-end call)."""

    def __init__(self, ctx, cfg: LayerCfg, max_rows: int):
        self.cfg = cfg
        self.handle = lib().m40host_layer_create(ctx, C.byref(cfg), max_rows)
        if not self.handle:
            raise RuntimeError(last_error())

    def forward_host(self, kv, weights: Weights, kvcfg: KvCfg, requests, x: np.ndarray, out: np.ndarray | None = None,
                     use_graph: bool = True) -> np.ndarray:
        n = len(requests)
        rid = np.array([r[0] for r in requests], np.uint64)
        sid = np.array([r[1] for r in requests], np.uint32)
        kvl = np.array([r[2] for r in requests], np.uint32)
        act = np.array([1 if r[3] else 0 for r in requests], np.uint32)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if out is None:
            out = np.empty_like(x)
        p = lambda a: a.ctypes.data_as(C.c_void_p)
        rc = lib().m40host_layer_forward_host(self.handle, kv, C.byref(weights), C.byref(kvcfg), n, p(rid), p(sid), p(kvl),
                                              p(act), p(x), p(out), 1 if use_graph else 0)
        if rc != 0:
            raise RuntimeError(f"layer forward failed rc={rc}: {last_error()}")
        return out

    def forward_host_raw(self, kv, weights, kvcfg, n, rid_p, sid_p, kvl_p, act_p, x_p, out_p, use_graph=True) -> int:
        return lib().m40host_layer_forward_host(self.handle, kv, C.byref(weights), C.byref(kvcfg), n, rid_p, sid_p, kvl_p,
                                                act_p, x_p, out_p, 1 if use_graph else 0)

    def forward_host_begin_raw(self, slot, kv, weights, kvcfg, n, rid_p, sid_p, kvl_p, act_p, x_p, use_graph=True) -> int:
        """First half of forward_host for slot 0 or 1: uploads on the prefill stream, enqueues the layer on the decode
        stream. Two slots may be in flight; end a slot before beginning it again."""
        return lib().m40host_layer_forward_host_begin(self.handle, slot, kv, C.byref(weights), C.byref(kvcfg), n, rid_p, sid_p,
                                                      kvl_p, act_p, x_p, 1 if use_graph else 0)

    def forward_host_end_raw(self, slot, out_p) -> int:
        """Second half: copies the slot's result to `out_p` (host) and returns when it has arrived."""
        return lib().m40host_layer_forward_host_end(self.handle, slot, out_p)

    def graph_replays(self) -> int:
        return int(lib().m40host_layer_graph_replays(self.handle))

    def close(self):
        if self.handle:
            lib().m40host_layer_destroy(self.handle)
            self.handle = None


class DecodeModel:
    """Greedy decode of a whole layer stack (embedding -> layers -> logits head -> arg-max on the device); mirror of the
    reference's session loop (src/decode_session.rs:637-954, src/infer/logits.rs:57-116, src/sampling.rs:95-108).
    `kv` is a dense cache with sequences * layers slots (slot = sequence * layers + layer, src/infer/kv.rs:109)."""

    def __init__(self, ctx, cfg: LayerCfg, layers, head: ModelHead, kv, sequences: int):
        arr = (Weights * len(layers))(*layers)
        self._keep = (arr, head, cfg)
        self.sequences, self.vocab = sequences, int(head.vocab)
        self.h = lib().m40host_model_create(ctx, C.byref(cfg), len(layers), arr, C.byref(head), kv, sequences)
        if not self.h:
            raise RuntimeError(last_error())

    def begin(self, token_ids, positions):
        t = np.ascontiguousarray(token_ids, dtype=np.uint32)
        p = np.ascontiguousarray(positions, dtype=np.uint32)
        assert t.shape == (self.sequences,) and p.shape == (self.sequences,)
        if lib().m40host_model_begin(self.h, t.ctypes.data_as(C.c_void_p), p.ctypes.data_as(C.c_void_p)) != 0:
            raise RuntimeError(last_error())

    def generate(self, steps: int, use_graph: bool = True, want_ids: bool = True, want_logits: bool = False):
        """Returns (ids [steps, sequences] or None, logits of the last step [sequences, vocab] or None)."""
        ids = np.empty((steps, self.sequences), np.uint32) if want_ids else None
        logits = np.empty((self.sequences, self.vocab), np.float32) if want_logits else None
        rc = lib().m40host_model_generate(self.h, steps, 1 if use_graph else 0,
                                          ids.ctypes.data_as(C.c_void_p) if want_ids else None,
                                          logits.ctypes.data_as(C.c_void_p) if want_logits else None)
        if rc != 0:
            raise RuntimeError(last_error())
        return ids, logits

    def graph_replays(self) -> int:
        return int(lib().m40host_model_graph_replays(self.h))

    def launches_per_step(self) -> int:
        return int(lib().m40host_model_launches_per_step(self.h))

    def close(self):
        if self.h:
            lib().m40host_model_destroy(self.h)
            self.h = None
