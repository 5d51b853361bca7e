"""Host-side description of a tree ensemble: the structure-of-arrays that crosses the C ABI.

The fields are the Treelite model fields cuML reads and writes when it hands a forest to its
inference library (reference: cpp/src/decisiontree/decisiontree.cuh:165-221,
cpp/src/randomforest/randomforest.cu:262-279, cpp/src/explainer/tree_shap.cu:268-300).  Importers
(sklearn, Treelite JSON dump, XGBoost JSON, LightGBM text, synthetic generators) all produce a
`ForestDesc`; `b2fil_forest_create` validates, packs and uploads it.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

# enums of include/b2fil.h
F32, F64 = 0, 1
NODE_LEAF, NODE_NUMERICAL, NODE_CATEGORICAL = 0, 1, 2
OP_LT, OP_LE, OP_GT, OP_GE = 0, 1, 2, 3
LAYOUTS = {"depth_first": 0, "breadth_first": 1, "layered": 2}
STORAGES = {"auto": 0, "dense": 1, "sparse": 2}
INFER_DEFAULT, INFER_PER_TREE, INFER_LEAF_ID, INFER_CLASS, INFER_PROBA2 = 0, 1, 2, 3, 4
POSTPROCS = {
    "identity": 0,
    "identity_multiclass": 0,
    "sigmoid": 1,
    "exponential": 2,
    "logarithm_one_plus_exp": 3,
    "signed_square": 4,
    "hinge": 5,
    "softmax": 6,
    "multiclass_ova": 7,
    "exponential_standard_ratio": 8,
}


class CForestDesc(C.Structure):
    """ctypes mirror of `b2fil_forest_desc`."""

    _fields_ = [
        ("n_trees", C.c_int32),
        ("n_features", C.c_int32),
        ("n_outputs", C.c_int32),
        ("leaf_vector_len", C.c_int32),
        ("tree_offsets", C.c_void_p),
        ("node_kind", C.c_void_p),
        ("feature", C.c_void_p),
        ("threshold", C.c_void_p),
        ("left", C.c_void_p),
        ("right", C.c_void_p),
        ("default_left", C.c_void_p),
        ("op", C.c_void_p),
        ("op_all", C.c_int32),
        ("cat_ptr", C.c_void_p),
        ("cat_values", C.c_void_p),
        ("cat_right", C.c_void_p),
        ("leaf_value", C.c_void_p),
        ("class_id", C.c_void_p),
        ("average_tree_output", C.c_int32),
        ("base_scores", C.c_void_p),
        ("postproc", C.c_int32),
        ("sigmoid_alpha", C.c_double),
        ("ratio_c", C.c_double),
    ]


class CCreateOpts(C.Structure):
    """ctypes mirror of `b2fil_create_opts`."""

    _fields_ = [
        ("precision", C.c_int32),
        ("layout", C.c_int32),
        ("storage", C.c_int32),
        ("align_bytes", C.c_int32),
        ("device_id", C.c_int32),
        ("default_chunk_size", C.c_int32),
        ("row_quantization", C.c_int32),
        ("compact_image", C.c_int32),
    ]


class CInfo(C.Structure):
    """ctypes mirror of `b2fil_info`."""

    _fields_ = [
        ("precision", C.c_int32),
        ("layout", C.c_int32),
        ("storage", C.c_int32),
        ("device_id", C.c_int32),
        ("n_trees", C.c_int32),
        ("n_features", C.c_int32),
        ("n_outputs", C.c_int32),
        ("leaf_vector_len", C.c_int32),
        ("max_depth", C.c_int32),
        ("dense_depth", C.c_int32),
        ("node_bytes", C.c_int32),
        ("has_categorical", C.c_int32),
        ("n_nodes_in", C.c_int64),
        ("n_nodes_packed", C.c_int64),
        ("device_bytes", C.c_int64),
        ("default_chunk_size", C.c_int32),
        ("row_quantization", C.c_int32),
        ("peer_direct", C.c_int32),
        ("clone_src_device", C.c_int32),
        ("compact_image", C.c_int32),
        ("top_levels", C.c_int32),
        ("scratch_pool_bytes", C.c_int64),
    ]


def _arr(a, dtype):
    if a is None:
        return None
    return np.ascontiguousarray(a, dtype=dtype)


@dataclass
class ForestDesc:
    """A tree ensemble as flat host arrays.

    Nodes of tree ``t`` occupy ``tree_offsets[t]:tree_offsets[t+1]``; the first of them is the
    root; ``left`` / ``right`` are indices relative to the tree's first node and that relative
    index is the node's id for ``apply``.
    """

    n_features: int
    n_outputs: int
    tree_offsets: np.ndarray
    node_kind: np.ndarray
    feature: np.ndarray
    threshold: np.ndarray
    left: np.ndarray
    right: np.ndarray
    default_left: np.ndarray
    leaf_value: np.ndarray
    leaf_vector_len: int = 1
    op: Optional[np.ndarray] = None
    op_all: int = OP_LT
    cat_ptr: Optional[np.ndarray] = None
    cat_values: Optional[np.ndarray] = None
    cat_right: Optional[np.ndarray] = None
    class_id: Optional[np.ndarray] = None
    average_tree_output: bool = False
    base_scores: Optional[np.ndarray] = None
    postproc: str = "identity"
    sigmoid_alpha: float = 1.0
    ratio_c: float = 1.0
    is_classifier: bool = False
    native_precision: str = "double"
    _keep: list = field(default_factory=list, repr=False)

    def __post_init__(self):
        self.tree_offsets = _arr(self.tree_offsets, np.int64)
        self.node_kind = _arr(self.node_kind, np.uint8)
        self.feature = _arr(self.feature, np.int32)
        self.threshold = _arr(self.threshold, np.float64)
        self.left = _arr(self.left, np.int32)
        self.right = _arr(self.right, np.int32)
        self.default_left = _arr(self.default_left, np.uint8)
        self.leaf_value = _arr(self.leaf_value, np.float64)
        self.op = _arr(self.op, np.uint8)
        self.cat_ptr = _arr(self.cat_ptr, np.int64)
        self.cat_values = _arr(self.cat_values, np.uint32)
        self.cat_right = _arr(self.cat_right, np.uint8)
        self.class_id = _arr(self.class_id, np.int32)
        self.base_scores = _arr(self.base_scores, np.float64)
        if self.postproc not in POSTPROCS:
            raise ValueError(f"unknown postprocessor {self.postproc!r}")

    @property
    def n_trees(self) -> int:
        return int(self.tree_offsets.shape[0] - 1)

    @property
    def n_nodes(self) -> int:
        return int(self.tree_offsets[-1])

    def to_c(self) -> CForestDesc:
        """Build the C struct; the arrays it points to stay owned by this object."""

        def p(a):
            return None if a is None else a.ctypes.data

        if self.cat_ptr is not None and self.cat_values is None:
            self.cat_values = np.zeros(1, np.uint32)
        d = CForestDesc()
        d.n_trees = self.n_trees
        d.n_features = int(self.n_features)
        d.n_outputs = int(self.n_outputs)
        d.leaf_vector_len = int(self.leaf_vector_len)
        d.tree_offsets = p(self.tree_offsets)
        d.node_kind = p(self.node_kind)
        d.feature = p(self.feature)
        d.threshold = p(self.threshold)
        d.left = p(self.left)
        d.right = p(self.right)
        d.default_left = p(self.default_left)
        d.op = p(self.op)
        d.op_all = int(self.op_all)
        d.cat_ptr = p(self.cat_ptr)
        d.cat_values = p(self.cat_values)
        d.cat_right = p(self.cat_right)
        d.leaf_value = p(self.leaf_value)
        d.class_id = p(self.class_id)
        d.average_tree_output = 1 if self.average_tree_output else 0
        d.base_scores = p(self.base_scores)
        d.postproc = POSTPROCS[self.postproc]
        d.sigmoid_alpha = float(self.sigmoid_alpha)
        d.ratio_c = float(self.ratio_c)
        return d

    # -- serialisation (pickle support of ForestInference goes through these) --------------------
    _ARRAYS = ("tree_offsets", "node_kind", "feature", "threshold", "left", "right",
               "default_left", "leaf_value", "op", "cat_ptr", "cat_values", "cat_right",
               "class_id", "base_scores")
    _SCALARS = ("n_features", "n_outputs", "leaf_vector_len", "op_all", "average_tree_output",
                "postproc", "sigmoid_alpha", "ratio_c", "is_classifier", "native_precision")

    def to_dict(self) -> dict:
        out = {k: getattr(self, k) for k in self._SCALARS}
        for k in self._ARRAYS:
            out[k] = getattr(self, k)
        return out

    @classmethod
    def from_dict(cls, d: dict) -> "ForestDesc":
        return cls(**{k: d[k] for k in cls._SCALARS + cls._ARRAYS})


def concatenate(descs) -> ForestDesc:
    """Join several ensembles over the same features and outputs into one, tree lists appended.

    Counterpart of `treelite.Model.concatenate` as used when per-worker forests are merged before
    prediction (reference: python/cuml/cuml/dask/ensemble/base.py:153-175).
    """
    descs = list(descs)
    if not descs:
        raise ValueError("nothing to concatenate")
    a = descs[0]
    for d in descs[1:]:
        if (d.n_features, d.n_outputs, d.leaf_vector_len, d.postproc, d.average_tree_output) != (
                a.n_features, a.n_outputs, a.leaf_vector_len, a.postproc, a.average_tree_output):
            raise ValueError("forests differ in shape or postprocessing")
    offs = [np.zeros(1, np.int64)]
    total = 0
    for d in descs:
        offs.append(d.tree_offsets[1:] + total)
        total += d.n_nodes

    def cat(name, default=None, dtype=None):
        vals = [getattr(d, name) for d in descs]
        if all(v is None for v in vals):
            return None
        out = []
        for d, v in zip(descs, vals):
            out.append(v if v is not None else default(d))
        return np.concatenate(out)

    any_cat = any(d.cat_ptr is not None for d in descs)
    cat_ptr = cat_values = None
    if any_cat:
        ptrs, vals, base = [np.zeros(1, np.int64)], [], 0
        for d in descs:
            if d.cat_ptr is None:
                ptrs.append(np.full(d.n_nodes, base, np.int64))
            else:
                ptrs.append(d.cat_ptr[1:] + base)
                vals.append(d.cat_values[: int(d.cat_ptr[-1])])
                base += int(d.cat_ptr[-1])
        cat_ptr = np.concatenate(ptrs)
        cat_values = np.concatenate(vals) if vals else np.zeros(1, np.uint32)
    op = None
    if any(d.op is not None for d in descs) or any(d.op_all != a.op_all for d in descs):
        op = np.concatenate([d.op if d.op is not None else np.full(d.n_nodes, d.op_all, np.uint8)
                             for d in descs])
    class_id = None
    if any(d.class_id is not None for d in descs) or (a.leaf_vector_len == 1 and a.n_outputs > 1):
        parts = []
        for d in descs:
            parts.append(d.class_id if d.class_id is not None
                         else (np.arange(d.n_trees) % d.n_outputs).astype(np.int32))
        class_id = np.concatenate(parts)
    return ForestDesc(
        n_features=a.n_features, n_outputs=a.n_outputs, leaf_vector_len=a.leaf_vector_len,
        tree_offsets=np.concatenate(offs),
        node_kind=cat("node_kind"), feature=cat("feature"), threshold=cat("threshold"),
        left=cat("left"), right=cat("right"), default_left=cat("default_left"),
        leaf_value=cat("leaf_value"),
        op=op,
        op_all=a.op_all, cat_ptr=cat_ptr, cat_values=cat_values,
        cat_right=cat("cat_right", default=lambda d: np.ones(d.n_nodes, np.uint8)),
        class_id=class_id, average_tree_output=a.average_tree_output,
        base_scores=a.base_scores, postproc=a.postproc, sigmoid_alpha=a.sigmoid_alpha,
        ratio_c=a.ratio_c, is_classifier=a.is_classifier, native_precision=a.native_precision)
