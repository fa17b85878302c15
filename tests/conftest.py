import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


# The one-launch row attention is chosen by cache size in production (small caches only); the tests exercise the
# cluster kernel at every size. Read once by the library, so it is set before the first call.
os.environ.setdefault("M40LLM_FUSED_ROW_MAX_KV_MB", "4096")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def O():
    from oracle import oracle

    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def pkg():
    import helpers

    return helpers.load_package()


@pytest.fixture(scope="session")
def nat(pkg):
    """The native library plus one context on device 0 (GPU tests only)."""
    import helpers

    return helpers.Native(pkg.native.lib())
