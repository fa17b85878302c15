"""Shared test helpers: package loader, device buffers over the C ABI, tolerances, generators."""
from __future__ import annotations

import ctypes as C
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "m40-llm_b200")
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libm40llm_ref.so")
GOLDEN = os.path.join(ROOT, "tests", "golden")

# Parity tolerance for floating-point outputs: |a - e| <= ATOL + RTOL * |e|.
ATOL = 1e-3
RTOL = 2e-3
# Two block scores closer than this are a tie for the selection comparison.
TIE_EPS = 1e-6


def load_package():
    if "m40_llm_b200" in sys.modules:
        return sys.modules["m40_llm_b200"]
    spec = importlib.util.spec_from_file_location(
        "m40_llm_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["m40_llm_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def assert_close(actual, expected, atol=ATOL, rtol=RTOL, what=""):
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape, (actual.shape, expected.shape)
    assert np.all(np.isfinite(actual)), f"{what}: non-finite output"
    err = np.abs(actual - expected)
    bound = atol + rtol * np.abs(expected)
    bad = err > bound
    if bad.any():
        i = int(np.argmax(err - bound))
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{err.size} outside |a-e| <= {atol} + {rtol}|e|; worst at flat index {i}: "
            f"actual={actual.ravel()[i]!r} expected={expected.ravel()[i]!r} err={err.ravel()[i]:.3e}")


def assert_selection_matches(sel_actual, sel_expected, scores_f64, what=""):
    """Selected block sets must match exactly unless the symmetric difference only contains blocks
    whose exact score is within TIE_EPS of the cut-off (the lowest selected) score. Order is not compared."""
    a = set(int(b) for b in sel_actual if int(b) != 0xFFFFFFFF)
    e = set(int(b) for b in sel_expected if int(b) != 0xFFFFFFFF)
    assert len(a) == len(e), f"{what}: selected {len(a)} blocks, expected {len(e)}"
    if a == e:
        return
    cutoff = min(scores_f64[b] for b in e)
    for b in a ^ e:
        assert abs(scores_f64[b] - cutoff) <= TIE_EPS, (
            f"{what}: block {b} differs and is not a tie (score {scores_f64[b]!r}, cut-off {cutoff!r})")


# Device buffers and the context wrapper live in the package (the benchmark uses them too).
DevBuf = load_package().native.DevBuf
Native = load_package().native.Native


def load_reference_lib(pkg):
    """The reference project's own cuda/kernels.cu built for sm_100a (oracle/_ref), or None."""
    if not os.path.exists(REF_LIB):
        return None
    dll = C.CDLL(REF_LIB)
    sigs = pkg.native.parse_header()
    for name, (restype, argtypes) in sigs.items():
        try:
            fn = getattr(dll, name)
        except AttributeError:
            continue
        fn.restype = restype
        fn.argtypes = argtypes
    return dll


def rope_rows_np(x, heads, hd, positions, base, scale, layout):
    """Independent float64-angle-free restatement is not wanted here: this mirrors the f32 formula
    (tests/rmsnorm_rope.rs:43-76) with numpy float32 ops, per row position."""
    x = np.array(x, dtype=np.float32).reshape(len(positions), heads, hd).copy()
    half = hd // 2
    i = np.arange(half, dtype=np.float32)
    inv = np.power(np.float32(base), (np.float32(-2.0) * i / np.float32(hd)).astype(np.float32)).astype(np.float32)
    for r, pos in enumerate(positions):
        theta = (np.float32(pos) * np.float32(scale)) * inv
        c = np.cos(theta).astype(np.float32)
        s = np.sin(theta).astype(np.float32)
        if layout == 1:
            a = x[r, :, :half].copy()
            b = x[r, :, half:].copy()
            x[r, :, :half] = a * c - b * s
            x[r, :, half:] = a * s + b * c
        else:
            a = x[r, :, 0::2].copy()
            b = x[r, :, 1::2].copy()
            x[r, :, 0::2] = a * c - b * s
            x[r, :, 1::2] = a * s + b * c
    return x
