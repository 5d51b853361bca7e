"""ctypes wrapper of the CPU oracle.  TEST INFRASTRUCTURE: imported only by tests/,
__graft_entry__.smoke() and the CPU-baseline legs of bench.py."""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(_HERE))
from cuml_b200.fil._desc import (CForestDesc, F32, F64, INFER_CLASS, INFER_DEFAULT,  # noqa: E402
                                 INFER_LEAF_ID, INFER_PER_TREE, INFER_PROBA2, ForestDesc)

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "_build", "libfil_oracle.so")
        if not os.path.exists(path):
            from oracle.build import build  # compiles with gcc when sources are newer

            path = build()
        _lib = C.CDLL(path)
        for fn in (_lib.fil_oracle_predict, _lib.fil_oracle_predict_packed):
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(CForestDesc), C.c_int, C.c_int, C.c_void_p, C.c_int64,
                           C.c_int64, C.c_void_p, C.c_double, C.c_int]
    return _lib


def predict(desc: ForestDesc, X: np.ndarray, kind: int = INFER_DEFAULT, precision: str = "single",
            threshold: float = 0.5, n_threads: int | None = None, packed: bool = False) -> np.ndarray:
    """Run the oracle on host rows.  `precision` decides the compare and output type.
    `packed=True` takes the walk over packed node records with eight rows side by side (same
    results, several times faster: the CPU baseline of the benchmarks); tests use the plain walk."""
    dt = np.float32 if precision == "single" else np.float64
    X = np.ascontiguousarray(X, dtype=dt)
    n = X.shape[0]
    nt, k = desc.n_trees, desc.n_outputs
    if kind == INFER_LEAF_ID:
        out = np.empty((n, nt), np.uint32)
    elif kind == INFER_PER_TREE:
        out = np.empty((n, nt, k) if desc.leaf_vector_len > 1 else (n, nt), dt)
    elif kind == INFER_CLASS:
        out = np.empty((n,), np.int32)
    elif kind == INFER_PROBA2:
        out = np.empty((n, 2), dt)
    else:
        out = np.empty((n, k), dt)
    cd = desc.to_c()
    fn = lib().fil_oracle_predict_packed if packed else lib().fil_oracle_predict
    rc = fn(C.byref(cd), F32 if precision == "single" else F64, kind,
                                  X.ctypes.data, n, X.shape[1] if X.ndim == 2 else desc.n_features,
                                  out.ctypes.data, float(threshold),
                                  int(n_threads or os.cpu_count() or 1))
    if rc != 0:
        raise RuntimeError(f"oracle failed with code {rc}")
    return out
