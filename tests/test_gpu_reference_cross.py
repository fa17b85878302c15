"""On the GPU box: the reference project's own CUDA translation unit (cuda/kernels.cu, compiled unmodified for
sm_100a into oracle/_ref/ by `make -C oracle ref`) and this library run the same seeded cases through the same
C ABI; both are compared with each other and with the oracle. Skipped when the reference build is absent."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
from helpers import assert_close

pytestmark = pytest.mark.gpu

sys.path.insert(0, helpers.GOLDEN)


@pytest.fixture(scope="module")
def both(tmp_path_factory, pkg):
    if not os.path.exists(helpers.REF_LIB):
        pytest.skip("oracle/_ref/libm40llm_ref.so not built (needs the reference checkout at build time)")
    d = tmp_path_factory.mktemp("golden")
    outs = {}
    for which in ("ref", "mine"):
        path = os.path.join(d, which + ".npz")
        # separate processes: the two libraries export the same symbol names
        subprocess.check_call([sys.executable, os.path.join(helpers.GOLDEN, "make_golden.py"), "--lib", which, "--out", path])
        outs[which] = dict(np.load(path))
    return outs


def test_same_cases_same_answers(both):
    ref, mine = both["ref"], both["mine"]
    for name, r in ref.items():
        m = mine[name]
        if r.dtype in (np.uint16, np.uint32):  # cache bytes and selected block indices: bit-exact
            if name.endswith("/k_cache"):
                # RoPE'd K: device powf/sinf/cosf may differ in the last ulp between two builds -> compare as f16 values
                assert_close(m.view(np.float16).astype(np.float32), r.view(np.float16).astype(np.float32), atol=2e-3, what=name)
            else:
                assert np.array_equal(m, r), name
        elif name.startswith("rope_"):
            # device powf (reference) vs correctly rounded inverse frequency (this library): angle differs by
            # ~pos * 5e-7 rad; see test_oracle_golden.py
            import cases
            rows, heads, hd, past, base, layout = cases.ROPE_CASES[name]
            tol = 1e-4 + (past + rows) * 6e-7 * float(np.abs(cases.rope_inputs(name)).max())
            assert_close(m, r, atol=tol, rtol=0, what=name)
        else:
            assert_close(m, r, what=name)
