"""`ForestInference`: the estimator-style front of the B200 forest-inference library.

Mirrors the surface cuML uses from its inference library: models are created with
`load_from_treelite_model` (python/cuml/cuml/ensemble/randomforest_common.pyx:402-409), expose
`predict`, `predict_proba`, `predict_per_tree` (randomforestclassifier.py:337,388,
randomforest_common.pyx:652) and `forest.get_dtype()` (randomforestclassifier.py:333); `load`,
`load_from_sklearn`, `apply`, `optimize` and the `layout`, `chunk_size`, `precision` options are
the remaining members of the `cuml.fil.ForestInference` interface.  All computation happens in
libb2fil.so on the GPU; this file only validates, converts array types and forwards pointers.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Optional

import numpy as np

from . import _lib
from ._desc import (CCreateOpts, CInfo, F32, F64, INFER_CLASS, INFER_DEFAULT, INFER_LEAF_ID,
                    INFER_PER_TREE, INFER_PROBA2, LAYOUTS, STORAGES, ForestDesc)

_PRECISIONS = ("single", "double", "native")


def _torch():
    import torch

    return torch


class _Forest:
    """Owner of one `b2fil_forest` handle (one device)."""

    def __init__(self, handle: int):
        self.handle = C.c_void_p(handle)
        info = CInfo()
        _lib.check(_lib.load().b2fil_forest_info(self.handle, C.byref(info)))
        self.info = info

    @classmethod
    def create(cls, desc: ForestDesc, precision: int, layout: int, storage: int,
               align_bytes: int, device_id: int, default_chunk_size: int,
               row_quantization: int = 0, compact_image: int = 0) -> "_Forest":
        lib = _lib.load()
        cd = desc.to_c()
        opts = CCreateOpts(precision, layout, storage, align_bytes, device_id, default_chunk_size,
                           row_quantization, compact_image)
        out = C.c_void_p()
        _lib.check(lib.b2fil_forest_create(C.byref(cd), C.byref(opts), C.byref(out)))
        return cls(out.value)

    def clone_to(self, device_id: int) -> "_Forest":
        out = C.c_void_p()
        _lib.check(_lib.load().b2fil_forest_clone_to_device(self.handle, device_id, C.byref(out)))
        return _Forest(out.value)

    def get_dtype(self):
        """dtype callers must cast inputs to (randomforestclassifier.py:333)."""
        return np.float32 if self.info.precision == F32 else np.float64

    def close(self):
        if self.handle:
            _lib.load().b2fil_forest_free(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ForestInference:
    """GPU inference for tree ensembles (gradient-boosted trees, random forests).

    Parameters mirror `cuml.fil.ForestInference`:

    layout : 'depth_first' | 'breadth_first' | 'layered' - node order of sparse storage.
    default_chunk_size : rows-per-CTA knob (1 -> 32 rows, 2 -> 64, >= 4 -> 128); None = automatic.
    align_bytes : pad every tree of a sparse forest to a multiple of this many bytes.
    precision : 'single' | 'double' | 'native' (the model's own threshold type).
    is_classifier : whether `predict` returns classes and `predict_proba` is available.
    storage : 'auto' | 'dense' | 'sparse' - 'dense' pads trees to complete binary trees with
        implicit child indexing; 'auto' chooses it for shallow forests.
    quantize_rows : dense forests (categorical splits only with categories below 32) predict on
        16-bit per-feature ranks of the inputs (exact: rank(x) <= j  <=>  x < threshold_j); False
        keeps the raw values.
    compact_nodes : sparse forests also get a compact image (8-byte internal nodes in depth-first
        order, leaves apart, the top levels of every tree as a heap that the kernel keeps in
        shared memory) whenever their fields fit; False keeps only the plain node array.
    device_id : CUDA device that holds the forest.
    output_type : 'input' (same kind of array as X), 'numpy' or 'torch'.
    """

    def __init__(self, *, treelite_model=None, handle=None, output_type: Optional[str] = None,
                 verbose=False, is_classifier: Optional[bool] = None, layout: str = "depth_first",
                 default_chunk_size: Optional[int] = None, align_bytes: Optional[int] = None,
                 precision: str = "single", device_id: int = 0, storage: str = "auto",
                 quantize_rows: bool = True, compact_nodes: bool = True):
        if layout not in LAYOUTS:
            raise ValueError(f"layout must be one of {sorted(LAYOUTS)}, got {layout!r}")
        if precision not in _PRECISIONS:
            raise ValueError(f"precision must be one of {_PRECISIONS}, got {precision!r}")
        if storage not in STORAGES:
            raise ValueError(f"storage must be one of {sorted(STORAGES)}, got {storage!r}")
        if default_chunk_size is not None and (default_chunk_size < 1 or
                                               default_chunk_size & (default_chunk_size - 1)):
            raise ValueError("default_chunk_size must be a positive power of two")
        self.layout = layout
        self.default_chunk_size = default_chunk_size
        self.align_bytes = align_bytes
        self.precision = precision
        self.device_id = int(device_id)
        self.storage = storage
        self.quantize_rows = bool(quantize_rows)
        self.compact_nodes = compact_nodes if isinstance(compact_nodes, int) else bool(compact_nodes)
        self.output_type = output_type or "input"
        self.verbose = verbose
        self.handle = handle
        self._desc: Optional[ForestDesc] = None
        self._forest: Optional[_Forest] = None
        self.is_classifier = bool(is_classifier) if is_classifier is not None else None
        if treelite_model is not None:
            self._set_model(treelite_model)

    # -- construction ---------------------------------------------------------------------------
    def _set_model(self, model):
        from .loaders import to_forest_desc

        desc = to_forest_desc(model)
        if self.is_classifier is None:
            self.is_classifier = bool(desc.is_classifier)
        self._desc = desc
        self._build()

    def _build(self):
        desc = self._desc
        prec = self.precision
        if prec == "native":
            prec = desc.native_precision
        self._forest = _Forest.create(
            desc, F32 if prec == "single" else F64, LAYOUTS[self.layout], STORAGES[self.storage],
            int(self.align_bytes or 0), self.device_id, int(self.default_chunk_size or 0),
            0 if self.quantize_rows else 1, self._compact_option())
        self._cache_facts()

    def _compact_option(self) -> int:
        """`compact_image` of the create options: True / False, or an int = at most that many
        heap levels (tuning aid)."""
        c = getattr(self, "compact_nodes", True)
        if isinstance(c, bool):
            return 0 if c else 1
        return 100 + int(c)

    def _cache_facts(self):
        """Plain-Python copies of what every call needs (ctypes field reads are slow)."""
        i = self._forest.info
        self._nf, self._nt, self._k = int(i.n_features), int(i.n_trees), int(i.n_outputs)
        self._vec = int(i.leaf_vector_len) > 1
        self._dev = int(i.device_id)
        self._np_dt = np.float32 if i.precision == F32 else np.float64
        self._torch_dt = None  # filled on the first device call (torch is imported lazily)

    @classmethod
    def load_from_treelite_model(cls, tl_model, **kwargs) -> "ForestInference":
        """Create from a Treelite-style model: a `ForestDesc`, an object with `dump_as_json()`
        (a `treelite.Model`), or the JSON dump itself."""
        kwargs.pop("device", None)
        is_clf = kwargs.pop("is_classifier", None)
        obj = cls(is_classifier=is_clf, **kwargs)
        obj._set_model(tl_model)
        return _specialise(obj)

    @classmethod
    def load_from_sklearn(cls, skl_model, **kwargs) -> "ForestInference":
        """Create from a fitted scikit-learn forest (random forest, extra trees, gradient
        boosting, single tree, isolation forest)."""
        from .importers import from_sklearn

        return cls.load_from_treelite_model(from_sklearn(skl_model), **kwargs)

    @classmethod
    def load(cls, path, *, model_type: Optional[str] = None, **kwargs) -> "ForestInference":
        """Create from a model file: XGBoost JSON ('xgboost_json') or UBJSON ('xgboost_ubjson',
        *.ubj), LightGBM text ('lightgbm'), Treelite JSON dump ('treelite_json') or a saved
        forest description ('b2fil_npz').  Without `model_type` the file extension decides."""
        from .loaders import load_file

        return cls.load_from_treelite_model(load_file(path, model_type), **kwargs)

    # -- properties -----------------------------------------------------------------------------
    @property
    def forest(self) -> _Forest:
        if self._forest is None:
            raise RuntimeError("no model loaded")
        return self._forest

    @property
    def n_outputs(self) -> int:
        return self._k if self._forest is not None else int(self.forest.info.n_outputs)

    @property
    def n_trees(self) -> int:
        return int(self.forest.info.n_trees)

    @property
    def n_features(self) -> int:
        return int(self.forest.info.n_features)

    def check_status(self) -> None:
        """Wait for all work on the forest's device and raise `B2FilError` (code -7) if a
        bounded wait inside a prediction kernel ran out since the last check.  Device-array
        predictions are stream ordered and do not check this themselves; host-array and sharded
        predictions do."""
        st = C.c_int32(0)
        _lib.check(_lib.load().b2fil_forest_status(self.forest.handle, C.byref(st)))

    def describe(self) -> dict:
        """Facts about the packed forest (storage chosen, node size, device bytes...)."""
        i = CInfo()  # asked again on every call: the scratch pool's size changes over time
        _lib.check(_lib.load().b2fil_forest_info(self.forest.handle, C.byref(i)))
        return {n: getattr(i, n) for n, _ in CInfo._fields_ if n != "reserved"}

    # -- pickling: the device forest is dropped and rebuilt on load
    #    (python/cuml/cuml/ensemble/randomforest_common.pyx:348-355) -----------------------------
    def __getstate__(self):
        st = dict(self.__dict__)
        st["_forest"] = None
        st["handle"] = None
        st["_desc"] = self._desc.to_dict() if self._desc is not None else None
        return st

    def __setstate__(self, st):
        self.__dict__.update(st)
        self._torch_dt = None
        if st.get("_desc") is not None:
            self._desc = ForestDesc.from_dict(st["_desc"])
            self._build()

    # -- prediction -----------------------------------------------------------------------------
    def _out_spec(self, kind: int, n: int):
        k, nt, dt = self._k, self._nt, self._np_dt
        if kind == INFER_LEAF_ID:
            return (n, nt), np.int32
        if kind == INFER_CLASS:
            return (n,), np.int32
        if kind == INFER_PROBA2:
            return (n, 2), dt
        if kind == INFER_PER_TREE:
            return ((n, nt, k) if self._vec else (n, nt)), dt
        return (n, k), dt

    def _run(self, X, kind: int, chunk_size: Optional[int], threshold: float = 0.5, preds=None):
        lib = _lib.load()
        f = self.forest
        dt = self._np_dt
        cs = int(chunk_size or self.default_chunk_size or 0)
        if cs and (cs < 1 or cs & (cs - 1)):
            raise ValueError("chunk_size must be a positive power of two")
        torch = None
        is_torch = False
        if not isinstance(X, np.ndarray):
            torch = _torch()
            if isinstance(X, torch.Tensor):
                is_torch = True
            elif hasattr(X, "__cuda_array_interface__"):
                X = torch.as_tensor(X, device=f"cuda:{self._dev}")
                is_torch = True
            else:
                X = np.asarray(X)
        if X.ndim == 1:
            X = X.reshape(1, -1)
        if X.ndim != 2 or X.shape[1] != self._nf:
            raise ValueError(f"X must have shape (n_rows, {self._nf}), got {tuple(X.shape)}")
        n = int(X.shape[0])
        shape, odt = self._out_spec(kind, n)
        want = self.output_type
        if is_torch and X.is_cuda:
            # device path: cast / make row-major like check_inputs(order="C") of the reference
            # (python/cuml/cuml/ensemble/randomforestclassifier.py:330-336)
            if self._torch_dt is None:
                self._torch_dt = {np.float32: torch.float32, np.float64: torch.float64,
                                  np.int32: torch.int32}
            tdt = self._torch_dt[dt]
            if X.get_device() != self._dev:
                raise ValueError(f"X is on {X.device}, the forest on cuda:{self._dev}")
            Xd = X if X.dtype == tdt else X.to(tdt)
            if Xd.stride(1) != 1:
                Xd = Xd.contiguous()
            todt = self._torch_dt[odt]
            if preds is not None:
                out = preds
                if (not isinstance(out, torch.Tensor) or tuple(out.shape) != shape or
                        out.dtype != todt or not out.is_contiguous()):
                    raise ValueError("preds has the wrong type, shape, dtype or layout")
            else:
                out = torch.empty(shape, dtype=todt, device=X.device)
            # the library makes the forest's device current itself; only the stream is needed
            stream = torch.cuda.current_stream(X.device).cuda_stream
            rc = lib.b2fil_predict(f.handle, kind, Xd.data_ptr(), n, Xd.stride(0),
                                   out.data_ptr(), cs, float(threshold), stream)
            if rc != 0:
                _lib.check(rc)
            if want == "numpy":
                return out.cpu().numpy()
            return out
        # host path
        if is_torch:
            Xh = X.detach().numpy()
        else:
            Xh = X
        Xh = np.ascontiguousarray(Xh, dtype=dt)
        if preds is not None and isinstance(preds, np.ndarray):
            out = preds
            if out.shape != shape or out.dtype != odt or not out.flags.c_contiguous:
                raise ValueError("preds has the wrong shape, dtype or layout")
        else:
            out = np.empty(shape, odt)
        _lib.check(lib.b2fil_predict_host(f.handle, kind, Xh.ctypes.data, n, Xh.shape[1],
                                          out.ctypes.data, cs, float(threshold)))
        if want == "torch" or (want == "input" and is_torch):
            return _torch().from_numpy(out)
        return out

    def predict_proba(self, X, *, preds=None, chunk_size: Optional[int] = None):
        """Class probabilities, shape (n_rows, n_classes).  A one-score binary model returns
        [1 - p, p]."""
        if not self.is_classifier:
            raise RuntimeError("predict_proba is only available for classifiers")
        kind = INFER_PROBA2 if self.n_outputs == 1 else INFER_DEFAULT
        return self._run(X, kind, chunk_size, preds=preds)

    def predict(self, X, *, preds=None, chunk_size: Optional[int] = None,
                threshold: Optional[float] = None):
        """Classifiers: class index per row (argmax, or `score > threshold` for binary models,
        default 0.5; randomforestclassifier.py:298,337).  Regressors: values, shape
        (n_rows, n_outputs) (randomforestregressor.py:269-275)."""
        if not self.is_classifier:
            return self._run(X, INFER_DEFAULT, chunk_size, preds=preds)
        if self.n_outputs == 2 and threshold is not None and float(threshold) != 0.5:
            proba = self._run(X, INFER_DEFAULT, chunk_size)
            res = proba[:, 1] > threshold
            return res.astype(np.int32) if isinstance(res, np.ndarray) else res.to(_torch().int32)
        return self._run(X, INFER_CLASS, chunk_size,
                         threshold=0.5 if threshold is None else float(threshold), preds=preds)

    def predict_per_tree(self, X, *, preds=None, chunk_size: Optional[int] = None):
        """Raw output of every tree: (n_rows, n_trees) or (n_rows, n_trees, n_classes)
        (randomforest_common.pyx:649-652)."""
        return self._run(X, INFER_PER_TREE, chunk_size, preds=preds)

    def apply(self, X, *, preds=None, chunk_size: Optional[int] = None):
        """Id of the leaf each row reaches in every tree, shape (n_rows, n_trees).  Ids are the
        node numbers of the imported model (scikit-learn's `tree_.apply` numbering for sklearn
        models)."""
        return self._run(X, INFER_LEAF_ID, chunk_size, preds=preds)

    def capture_graph(self, batch_size: int, predict_method: str = "predict"):
        """Record `predict_method` for device batches of exactly `batch_size` rows as a CUDA
        graph; returns a `GraphedPredictor` to call with such batches (small-batch serving)."""
        return _capture(self, int(batch_size), predict_method)

    def optimize(self, *, data=None, batch_size: int = 1024, unique_batches: int = 10,
                 timeout: float = 0.2, predict_method: str = "predict",
                 max_chunk_size: Optional[int] = None, seed: int = 0, layouts=None):
        """Time `predict_method` on device batches for every chunk size and keep the fastest as
        the default chunk size; returns it.

        `layouts`: node orders to try as well (the reference's tests sweep all three,
        python/cuml/tests/test_random_forest.py:902-1024).  The node order only matters to
        forests that run the plain sparse kernel, so by default (None) the sweep covers the three
        orders exactly for those (sparse storage without a compact image) and is skipped
        otherwise; pass a list to force it.  Trying an order re-packs the forest from its
        description; the fastest (layout, chunk size) pair is kept and `self.layout` updated."""
        torch = _torch()
        dev = torch.device(f"cuda:{self.forest.info.device_id}")
        tdt = torch.float32 if self.forest.get_dtype() == np.float32 else torch.float64
        if data is None:
            g = torch.Generator(device=dev)
            g.manual_seed(seed)
            data = torch.randn((unique_batches, batch_size, self.n_features), generator=g,
                               device=dev, dtype=tdt)
        else:
            data = torch.as_tensor(data, device=dev, dtype=tdt)
            if data.ndim == 2:
                data = data.unsqueeze(0)

        def sweep_chunks():
            fn = getattr(self, predict_method)
            best, best_t = None, float("inf")
            for cs in (1, 2, 4, 8, 16, 32):
                if max_chunk_size is not None and cs > max_chunk_size:
                    break
                fn(data[0], chunk_size=cs)
                torch.cuda.synchronize(dev)
                t0, reps = time.perf_counter(), 0
                while True:
                    for b in range(data.shape[0]):
                        fn(data[b], chunk_size=cs)
                    torch.cuda.synchronize(dev)
                    reps += 1
                    if time.perf_counter() - t0 > timeout / 6 or reps >= 20:
                        break
                t = (time.perf_counter() - t0) / reps
                if t < best_t:
                    best, best_t = cs, t
            return best, best_t

        if layouts is None:
            d = self.describe()
            plain_sparse = d["storage"] == STORAGES["sparse"] and not d["compact_image"]
            layouts = list(LAYOUTS) if (plain_sparse and self._desc is not None) else []
        layouts = [l for l in layouts if l in LAYOUTS]
        if not layouts or self._desc is None:
            best, _ = sweep_chunks()
            self.default_chunk_size = best
            return best
        results = {}
        for layout in layouts:
            if layout != self.layout:
                self.layout = layout
                self._build()
            results[layout] = sweep_chunks()
        best_layout = min(results, key=lambda l: results[l][1])
        if best_layout != self.layout:
            self.layout = best_layout
            self._build()
        self.default_chunk_size = results[best_layout][0]
        return self.default_chunk_size


class GraphedPredictor:
    """A prediction of fixed batch size recorded once as a CUDA graph and replayed per call.

    Replaying skips the per-call launch work of the host, which is what bounds the latency of
    small batches.  `__call__` copies the rows into the graph's static input buffer, replays, and
    returns the static output tensor (overwritten by the next call)."""

    def __init__(self, graph, static_in, static_out):
        self.graph = graph
        self.static_in = static_in
        self.static_out = static_out

    def __call__(self, X):
        if tuple(X.shape) != tuple(self.static_in.shape):
            raise ValueError(f"this graph was recorded for input shape {tuple(self.static_in.shape)}")
        self.static_in.copy_(X)
        self.graph.replay()
        return self.static_out


def _capture(model: "ForestInference", batch_size: int, predict_method: str) -> GraphedPredictor:
    torch = _torch()
    dev = torch.device(f"cuda:{model._dev}")
    tdt = torch.float32 if model._np_dt == np.float32 else torch.float64
    fn = getattr(model, predict_method)
    static_in = torch.zeros((batch_size, model._nf), device=dev, dtype=tdt)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(3):  # first calls set kernel attributes and warm the scratch pool
            fn(static_in)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = fn(static_in)
    return GraphedPredictor(graph, static_in, static_out)


class ForestInferenceClassifier(ForestInference):
    """`ForestInference` whose model is a classifier."""


class ForestInferenceRegressor(ForestInference):
    """`ForestInference` whose model is a regressor."""


def _specialise(obj: ForestInference) -> ForestInference:
    obj.__class__ = ForestInferenceClassifier if obj.is_classifier else ForestInferenceRegressor
    return obj


def load_from_treelite_model(tl_model, device: str = "gpu", layout: str = "depth_first",
                             default_chunk_size: Optional[int] = None,
                             align_bytes: Optional[int] = None, handle=None, **kwargs):
    """Module-level constructor with the signature cuML calls
    (python/cuml/cuml/ensemble/randomforest_common.pyx:402-409).  Only device='gpu' exists."""
    if device != "gpu":
        raise ValueError("this library runs on the GPU only; device must be 'gpu'")
    return ForestInference.load_from_treelite_model(
        tl_model, layout=layout, default_chunk_size=default_chunk_size, align_bytes=align_bytes,
        handle=handle, **kwargs)
