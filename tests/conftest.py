import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def lib():
    """libb2fil.so, built on demand."""
    from cuml_b200 import build
    from cuml_b200.fil import _lib

    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def pack_check():
    """Test-only host walker over packed forests (tests/native/pack_check.cpp)."""
    import ctypes as C
    import subprocess

    from cuml_b200.fil._desc import CCreateOpts, CForestDesc

    src = os.path.join(ROOT, "tests", "native", "pack_check.cpp")
    pack = os.path.join(ROOT, "cuml_b200", "csrc", "pack.cpp")
    out_dir = os.path.join(ROOT, "tests", "native", "_build")
    os.makedirs(out_dir, exist_ok=True)
    so = os.path.join(out_dir, "libpack_check.so")
    deps = [src, pack, os.path.join(ROOT, "cuml_b200", "csrc", "forest.hpp")]
    if not os.path.exists(so) or any(os.path.getmtime(d) > os.path.getmtime(so) for d in deps):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-o", so, src, pack])
    lib = C.CDLL(so)
    lib.pack_check.restype = C.c_int
    lib.pack_check.argtypes = [C.POINTER(CForestDesc), C.POINTER(CCreateOpts), C.c_void_p,
                               C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.pack_check_error.restype = C.c_char_p
    return lib
