"""The shared library exports every symbol include/m40llm_native.h declares, and the header covers every symbol of
the reference's FFI block (src/cuda.rs:87-682; names listed in tests/golden/reference_ffi_symbols.txt, extracted by
tests/golden/extract_ffi_symbols.py). No compute calls: runs without a GPU."""
import ctypes as C
import os

import helpers


def test_library_exports_every_declared_symbol(pkg):
    sigs = pkg.native.parse_header()
    assert len(sigs) >= 100
    dll = C.CDLL(pkg.native.LIB_PATH)
    missing = [n for n in sigs if not hasattr(dll, n)]
    assert not missing, missing


def test_header_covers_reference_ffi(pkg):
    names = [l.strip() for l in open(os.path.join(helpers.GOLDEN, "reference_ffi_symbols.txt")) if l.strip()]
    assert len(names) == 73
    sigs = pkg.native.parse_header()
    assert not [n for n in names if n not in sigs]


def test_argument_checks_need_no_device(pkg):
    """Null handles are rejected before any CUDA call (rc -1 as in the reference, cuda/kernels.cu:1056, 3887)."""
    L = pkg.native.lib()
    assert L.m40llm_rms_norm_f32_async(None, None, None, 1, 8, 1e-5) == -1
    assert L.m40llm_attention_last_token_f32_gqa_async(None, None, 0, None, 8, 1, None) == -1
    assert L.m40llm_residual_add_f32_async(None, None, None, None, 4) == -1
    assert L.m40llm_start_persistent_decode(None) == -1
    assert L.m40llm_kvcache_create(None, 8, 1, 1, 8) is None
