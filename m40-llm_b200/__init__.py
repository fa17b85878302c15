"""B200-native drop-in for the m40-llm decode hot path.

``native`` binds the C ABI (libm40llm_native.so); ``host`` binds the C++ mirror of the reference
host's decode-layer driver, which sits on top of that ABI. The package name carries a hyphen (it is the repo's
directory name), so harnesses load it by path:

    spec = importlib.util.spec_from_file_location("m40_llm_b200", ".../m40-llm_b200/__init__.py",
                                                  submodule_search_locations=[".../m40-llm_b200"])
"""
from . import host, native  # noqa: F401


def __getattr__(name):
    # `splitk` needs torch.distributed; loaded on first use so that the ctypes-only modules import without torch.
    if name == "splitk":
        import importlib
        return importlib.import_module(".splitk", __name__)
    raise AttributeError(name)
