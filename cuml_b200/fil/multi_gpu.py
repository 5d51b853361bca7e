"""Row-sharded prediction over the GPUs of one box, from a single process.

The forest is replicated into every GPU's own memory and the batch is split into contiguous row
shards; each shard is predicted where it lives and the results are gathered on the first device by
peer copies.  Nothing is reduced across GPUs, so no collective library is involved.  This is the
arrangement of the reference's Dask path (model broadcast to every worker, row partitions
predicted by the worker that holds them, results concatenated by rows:
python/cuml/cuml/dask/ensemble/base.py:153-175,210-218, python/cuml/cuml/dask/common/base.py:276-316).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._desc import INFER_CLASS, INFER_DEFAULT, INFER_LEAF_ID, INFER_PER_TREE, INFER_PROBA2
from .forest_inference import ForestInference


def shard_rows(n_rows: int, n_shards: int) -> List[Tuple[int, int]]:
    """Contiguous row ranges [begin, end) of `n_shards` shards that differ by at most one row;
    shard g covers rows [g*N/G, (g+1)*N/G)."""
    if n_shards < 1:
        raise ValueError("n_shards must be at least 1")
    if n_rows < 0:
        raise ValueError("n_rows must not be negative")
    return [((g * n_rows) // n_shards, ((g + 1) * n_rows) // n_shards) for g in range(n_shards)]


class ShardedForestInference:
    """A `ForestInference` replicated on several devices of one box."""

    def __init__(self, model: ForestInference, device_ids: Sequence[int]):
        if not device_ids:
            raise ValueError("device_ids must not be empty")
        if len(set(device_ids)) != len(device_ids):
            raise ValueError("device_ids must be distinct")
        if model.forest.info.device_id != device_ids[0]:
            raise ValueError("the model must live on the first device of device_ids")
        self.model = model
        self.device_ids = list(device_ids)
        self._lib = _lib.load()
        self._forests = [model.forest] + [model.forest.clone_to(d) for d in device_ids[1:]]

    def last_timing(self) -> dict:
        """Device-side times of this thread's last sharded call (`b2fil_last_sharded_timing`):
        the slowest device's kernels, the slowest gather copy, the host's wall time from the
        first launch to the last device done, and whether the gather went over direct peer
        paths."""
        c, g, w = C.c_double(), C.c_double(), C.c_double()
        d = C.c_int()
        _lib.check(self._lib.b2fil_last_sharded_timing(C.byref(c), C.byref(g), C.byref(w),
                                                       C.byref(d)))
        return {"compute_ms": c.value, "gather_ms": g.value, "wall_ms": w.value,
                "gather_direct": d.value}

    def _predict(self, shards, kind: int, chunk_size: Optional[int] = None, threshold=0.5,
                 preds=None):
        """`shards[i]` is a 2-d torch tensor on device i holding that device's rows.  `preds`, if
        given, is the output tensor on the first device (right shape and dtype, contiguous)."""
        import torch

        lib = _lib.load()
        n_dev = len(self.device_ids)
        if len(shards) != n_dev:
            raise ValueError(f"expected {n_dev} shards, got {len(shards)}")
        f0 = self._forests[0]
        dt = f0.get_dtype()
        tdt = torch.float32 if dt == np.float32 else torch.float64
        nf = f0.info.n_features
        prepared = []
        for dev, x in zip(self.device_ids, shards):
            if not isinstance(x, torch.Tensor) or not x.is_cuda or x.device.index != dev:
                raise ValueError(f"shard for device {dev} must be a CUDA tensor on that device")
            if x.ndim != 2 or x.shape[1] != nf:
                raise ValueError(f"every shard must have shape (rows, {nf})")
            if x.dtype != tdt:
                x = x.to(tdt)
            prepared.append(x if x.is_contiguous() else x.contiguous())
        rows = [int(x.shape[0]) for x in prepared]
        shape, odt = self.model._out_spec(kind, sum(rows))
        todt = {np.int32: torch.int32, np.float32: torch.float32, np.float64: torch.float64}[odt]
        if preds is not None:
            out = preds
            if (tuple(out.shape) != tuple(shape) or out.dtype != todt or not out.is_contiguous()
                    or out.device.index != self.device_ids[0]):
                raise ValueError("preds has the wrong shape, dtype, layout or device")
        else:
            out = torch.empty(shape, dtype=todt, device=f"cuda:{self.device_ids[0]}")
        for dev in self.device_ids:
            torch.cuda.synchronize(dev)  # inputs may still be in flight on the callers' streams
        handles = (C.c_void_p * n_dev)(*[f.handle for f in self._forests])
        xs = (C.c_void_p * n_dev)(*[x.data_ptr() for x in prepared])
        counts = (C.c_int64 * n_dev)(*rows)
        _lib.check(lib.b2fil_predict_sharded(handles, n_dev, kind, xs, counts, nf, out.data_ptr(),
                                             int(chunk_size or 0), float(threshold)))
        return out

    def predict_proba(self, shards, chunk_size=None, preds=None):
        kind = INFER_PROBA2 if self.model.n_outputs == 1 else INFER_DEFAULT
        return self._predict(shards, kind, chunk_size, preds=preds)

    def predict(self, shards, chunk_size=None, threshold=None):
        if not self.model.is_classifier:
            return self._predict(shards, INFER_DEFAULT, chunk_size)
        return self._predict(shards, INFER_CLASS, chunk_size,
                             0.5 if threshold is None else threshold)

    def apply(self, shards, chunk_size=None):
        return self._predict(shards, INFER_LEAF_ID, chunk_size)

    def predict_per_tree(self, shards, chunk_size=None):
        return self._predict(shards, INFER_PER_TREE, chunk_size)

    def scatter(self, X):
        """Split a host or device array into this object's row shards, one per device."""
        import torch

        X = torch.as_tensor(X)
        return [X[b:e].to(f"cuda:{d}", non_blocking=True)
                for (b, e), d in zip(shard_rows(X.shape[0], len(self.device_ids)),
                                     self.device_ids)]
