"""ctypes view of libm40llm_native.so with signatures derived from include/m40llm_native.h.

This is the harness-side stand-in for the reference's Rust FFI block (src/cuda.rs:87-682):
every exported `m40llm_*` function is reachable as ``lib.<name>(...)`` with ctypes argument
conversion taken from the C declaration. There is no CPU fallback: if the shared library is
missing the import fails, and every compute entry point needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libm40llm_native.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "m40llm_native.h")

ERR_UNSUPPORTED = -100
ERR_LIMIT = -101

_SCALARS = {
    "int": C.c_int, "uint32_t": C.c_uint32, "uint64_t": C.c_uint64, "size_t": C.c_size_t, "float": C.c_float,
}


def _ctype(decl: str):
    decl = decl.replace("const", " ").strip()
    if "*" in decl:
        return C.c_void_p
    base = decl.split()[0]
    return _SCALARS[base]


def parse_header(path: str = HEADER_PATH) -> dict[str, tuple[object, list[object]]]:
    """Returns {function name: (restype, [argtypes])} for every prototype in the header."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"#[^\n]*", " ", text)
    text = re.sub(r"typedef\s+struct\s*\{.*?\}\s*\w+\s*;", " ", text, flags=re.S)
    text = re.sub(r"typedef[^;]*;", " ", text)
    out = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(m40llm_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        restype = None if ret == "void" else _ctype(ret)
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                # drop the parameter name (last identifier) unless the declaration is just a type
                a = re.sub(r"\b\w+$", "", a).strip() if not a.endswith("*") else a
                argtypes.append(_ctype(a))
        out[name] = (restype, argtypes)
    return out


class NativeLib:
    """Loads the shared library and applies the header's signatures."""

    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python m40-llm_b200/build.py` (needs nvcc); there is no fallback")
        self._dll = C.CDLL(path)
        self.signatures = parse_header()
        for name, (restype, argtypes) in self.signatures.items():
            fn = getattr(self._dll, name)
            fn.restype = restype
            fn.argtypes = argtypes

    def __getattr__(self, name):
        return getattr(self._dll, name)


_lib = None


def lib() -> NativeLib:
    global _lib
    if _lib is None:
        _lib = NativeLib()
    return _lib


class DevBuf:
    """A device allocation made and moved through the C ABI (m40llm_device_malloc / memcpy_*)."""

    def __init__(self, nat: "Native", nbytes: int):
        self.nat = nat
        self.nbytes = max(int(nbytes), 4)
        p = C.c_void_p()
        rc = nat.lib.m40llm_device_malloc(nat.ctx, self.nbytes, C.byref(p))
        assert rc == 0 and p.value, f"device_malloc rc={rc}"
        self.ptr = p.value

    def upload(self, arr: np.ndarray):
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes
        if arr.nbytes:
            rc = self.nat.lib.m40llm_memcpy_h2d(self.nat.ctx, self.ptr, arr.ctypes.data_as(C.c_void_p), arr.nbytes)
            assert rc == 0, rc
        return self

    def download(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        if out.nbytes:
            rc = self.nat.lib.m40llm_memcpy_d2h(self.nat.ctx, out.ctypes.data_as(C.c_void_p), self.ptr, out.nbytes)
            assert rc == 0, rc
        return out

    def free(self):
        if self.ptr:
            self.nat.lib.m40llm_device_free(self.nat.ctx, self.ptr)
            self.ptr = None


class Native:
    """One context on a device plus conveniences for harnesses (tests, benchmark). `lib` may be this library or
    another build of the same ABI (the reference's own translation unit compiled for sm_100a)."""

    def __init__(self, lib, device: int = 0):
        self.lib = lib
        self.ctx = lib.m40llm_create_context(device)
        assert self.ctx, "m40llm_create_context failed (no CUDA device?)"
        self._bufs: list[DevBuf] = []

    def buf(self, arr_or_bytes) -> DevBuf:
        if isinstance(arr_or_bytes, (int, np.integer)):
            b = DevBuf(self, int(arr_or_bytes))
        else:
            arr = np.ascontiguousarray(arr_or_bytes)
            b = DevBuf(self, arr.nbytes).upload(arr)
        self._bufs.append(b)
        return b

    def sync(self, kind: int | None = None):
        for k in ((0, 1) if kind is None else (kind,)):
            rc = self.lib.m40llm_stream_synchronize(self.ctx, k)
            assert rc == 0, rc

    def free_all(self):
        for b in self._bufs:
            b.free()
        self._bufs.clear()

    # ---- KV cache conveniences -------------------------------------------------
    def kv_dense(self, max_seq, slots, kv_heads, hd):
        kv = self.lib.m40llm_kvcache_create(self.ctx, max_seq, slots, kv_heads, hd)
        assert kv, "kvcache_create failed"
        return kv

    def kv_compressed(self, max_seq, slots, kv_heads, hd, recent, block, top):
        kv = self.lib.m40llm_kvcache_create_compressed(self.ctx, max_seq, slots, kv_heads, hd, recent, block, top, 0, 0, 2)
        assert kv, "kvcache_create_compressed failed"
        return kv

    def kv_fill(self, kv, seq_id, k_f16, v_f16, final_len=None, tok_begin=0):
        """Bulk-load f16 K/V [tokens, kv_heads, hd] (K already rotated) through the harness loader."""
        k_f16 = np.ascontiguousarray(k_f16)
        v_f16 = np.ascontiguousarray(v_f16)
        n = k_f16.shape[0]
        rc = self.lib.m40llm_kvcache_debug_write_range(
            self.ctx, kv, seq_id, tok_begin, n, k_f16.ctypes.data_as(C.c_void_p), v_f16.ctypes.data_as(C.c_void_p),
            tok_begin + n if final_len is None else final_len)
        assert rc == 0, rc

    def kv_append_tokens(self, kv, seq_id, k_f32, v_f32, base=10000.0, scale=0.0, layout=0, start=0):
        """Token-by-token append through m40llm_kvcache_append_token_f32_rope_k_at_layout_async."""
        n = k_f32.shape[0]
        dk = self.buf(k_f32.astype(np.float32))
        dv = self.buf(v_f32.astype(np.float32))
        stride = k_f32[0].size * 4
        for t in range(n):
            rc = self.lib.m40llm_kvcache_append_token_f32_rope_k_at_layout_async(
                self.ctx, kv, seq_id, dk.ptr + t * stride, dv.ptr + t * stride, start + t, start + t, base, scale, layout)
            assert rc == 0, rc
        self.sync(1)
