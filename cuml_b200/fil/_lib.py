"""ctypes binding of libb2fil.so.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

from ._desc import CCreateOpts, CForestDesc, CInfo

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "lib", "libb2fil.so")

ERRORS = {-1: "invalid argument", -2: "bad forest", -3: "unsupported", -4: "CUDA error",
          -5: "out of memory", -6: "too large", -7: "timeout"}


class B2FilError(RuntimeError):
    """A libb2fil call returned an error code; `.code` holds it."""

    def __init__(self, code: int, message: str):
        super().__init__(f"b2fil error {code} ({ERRORS.get(code, '?')}): {message}")
        self.code = code


_lib = None


def load() -> C.CDLL:
    """Load libb2fil.so, building it with nvcc when it is missing or older than its sources."""
    global _lib
    if _lib is not None:
        return _lib
    from .. import build as _build

    if not _build.up_to_date():
        try:
            _build.build()
        except Exception:
            # a stale library on a box without nvcc is still loadable; a missing one is not
            if not os.path.exists(LIB_PATH):
                raise
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing and could not be built; "
                          "run `python -m cuml_b200.build`")
    lib = C.CDLL(LIB_PATH)
    vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int
    lib.b2fil_last_error.restype = C.c_char_p
    lib.b2fil_last_error.argtypes = []
    lib.b2fil_version.restype = i32
    lib.b2fil_kernel_launches.restype = i64
    lib.b2fil_forest_create.restype = i32
    lib.b2fil_forest_create.argtypes = [C.POINTER(CForestDesc), C.POINTER(CCreateOpts),
                                        C.POINTER(vp)]
    lib.b2fil_forest_clone_to_device.restype = i32
    lib.b2fil_forest_clone_to_device.argtypes = [vp, i32, C.POINTER(vp)]
    lib.b2fil_forest_free.restype = i32
    lib.b2fil_forest_free.argtypes = [vp]
    lib.b2fil_forest_info.restype = i32
    lib.b2fil_forest_info.argtypes = [vp, C.POINTER(CInfo)]
    lib.b2fil_forest_status.restype = i32
    lib.b2fil_forest_status.argtypes = [vp, C.POINTER(C.c_int32)]
    lib.b2fil_forest_selftest_timeout.restype = i32
    lib.b2fil_forest_selftest_timeout.argtypes = [vp, i32, vp]
    lib.b2fil_set_tuning.restype = i32
    lib.b2fil_set_tuning.argtypes = [C.c_char_p, i32]
    lib.b2fil_last_variant.restype = i32
    lib.b2fil_last_variant.argtypes = [C.c_char_p, C.c_size_t]
    lib.b2fil_enable_peer_access.restype = i32
    lib.b2fil_enable_peer_access.argtypes = [i32, i32]
    lib.b2fil_last_sharded_timing.restype = i32
    lib.b2fil_last_sharded_timing.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_double),
                                              C.POINTER(C.c_double), C.POINTER(i32)]
    lib.b2fil_output_elems_per_row.restype = i64
    lib.b2fil_output_elems_per_row.argtypes = [vp, i32]
    lib.b2fil_predict.restype = i32
    lib.b2fil_predict.argtypes = [vp, i32, vp, i64, i64, vp, i32, C.c_double, vp]
    lib.b2fil_predict_fixed_scratch.restype = i32
    lib.b2fil_predict_fixed_scratch.argtypes = [vp, i32, vp, i64, i64, vp, i32, C.c_double, vp]
    lib.b2fil_predict_host.restype = i32
    lib.b2fil_predict_host.argtypes = [vp, i32, vp, i64, i64, vp, i32, C.c_double]
    lib.b2fil_predict_sharded.restype = i32
    lib.b2fil_predict_sharded.argtypes = [C.POINTER(vp), i32, i32, C.POINTER(vp),
                                          C.POINTER(i64), i64, vp, i32, C.c_double]
    _lib = lib
    return lib


def last_variant() -> str:
    """Kernels the calling thread's most recent prediction enqueued (`b2fil_last_variant`)."""
    buf = C.create_string_buffer(512)
    load().b2fil_last_variant(buf, len(buf))
    return buf.value.decode()


def check(rc: int) -> None:
    if rc != 0:
        raise B2FilError(rc, load().b2fil_last_error().decode("utf-8", "replace"))
