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
