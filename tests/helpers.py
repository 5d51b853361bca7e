"""Shared test helpers: random ragged forests, a pure-Python evaluator, input generators."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from cuml_b200.fil._desc import (NODE_CATEGORICAL, NODE_LEAF, NODE_NUMERICAL, OP_GE, OP_GT, OP_LE,
                                 OP_LT, CCreateOpts, ForestDesc, LAYOUTS, STORAGES)


def random_forest_desc(seed, n_trees=7, n_features=6, max_depth=5, n_outputs=1, vector=False,
                       categorical=False, big_categories=False, mixed_ops=False, op=OP_LT,
                       postproc="identity", average=False, p_leaf=0.25, base=False,
                       integer_thresholds=False):
    """Random ragged forest.  Node 0 of each tree is the root; nodes are numbered in creation
    (pre-order) order, so left/right are arbitrary relative indices."""
    rng = np.random.default_rng(seed)
    kind, feat, thr, left, right, dl, opv, leaf = [], [], [], [], [], [], [], []
    cat_lists, cat_right = [], []
    offs = [0]
    width = n_outputs if vector else 1
    for _ in range(n_trees):
        base_idx = len(kind)

        def new_node():
            kind.append(NODE_LEAF)
            feat.append(0)
            thr.append(0.0)
            left.append(-1)
            right.append(-1)
            dl.append(0)
            opv.append(op)
            leaf.append(np.zeros(width))
            cat_lists.append([])
            cat_right.append(1)
            return len(kind) - 1 - base_idx

        def grow(rel, depth):
            g = base_idx + rel
            if depth >= max_depth or (depth > 0 and rng.random() < p_leaf):
                leaf[g] = rng.standard_normal(width).astype(np.float32).astype(np.float64)
                return
            feat[g] = int(rng.integers(0, n_features))
            dl[g] = int(rng.integers(0, 2))
            if categorical and rng.random() < 0.4:
                kind[g] = NODE_CATEGORICAL
                hi = 70 if big_categories else 20
                n_c = int(rng.integers(0, 6))
                cat_lists[g] = sorted(set(int(c) for c in rng.integers(0, hi, size=n_c)))
                cat_right[g] = int(rng.integers(0, 2))
            else:
                kind[g] = NODE_NUMERICAL
                if integer_thresholds:
                    thr[g] = float(rng.integers(-2, 3))
                else:
                    thr[g] = float(np.float32(rng.standard_normal()))
                if mixed_ops:
                    opv[g] = int(rng.integers(0, 4))
            # create children in random order so that relative indices are not monotone
            if rng.random() < 0.5:
                l = new_node(); r = new_node()
            else:
                r = new_node(); l = new_node()
            left[g], right[g] = l, r
            grow(l, depth + 1)
            grow(r, depth + 1)

        root = new_node()
        grow(root, 0)
        offs.append(len(kind))
    n = len(kind)
    cat_ptr = cat_values = cr = None
    if categorical:
        counts = [len(c) for c in cat_lists]
        cat_ptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        cat_values = np.asarray([c for l in cat_lists for c in l] or [0], np.uint32)
        cr = np.asarray(cat_right, np.uint8)
    class_id = None
    if not vector and n_outputs > 1:
        class_id = rng.integers(0, n_outputs, size=n_trees).astype(np.int32)
    return ForestDesc(
        n_features=n_features, n_outputs=n_outputs, leaf_vector_len=width,
        tree_offsets=np.asarray(offs, np.int64), node_kind=np.asarray(kind, np.uint8),
        feature=np.asarray(feat, np.int32), threshold=np.asarray(thr, np.float64),
        left=np.asarray(left, np.int32), right=np.asarray(right, np.int32),
        default_left=np.asarray(dl, np.uint8), leaf_value=np.concatenate(leaf),
        op=np.asarray(opv, np.uint8) if mixed_ops else None, op_all=op, cat_ptr=cat_ptr,
        cat_values=cat_values, cat_right=cr, class_id=class_id, average_tree_output=average,
        base_scores=(rng.standard_normal(n_outputs) if base else None), postproc=postproc,
        sigmoid_alpha=1.5 if postproc in ("sigmoid", "multiclass_ova") else 1.0, ratio_c=2.0,
        is_classifier=n_outputs > 1 or postproc == "sigmoid")


def random_rows(seed, n_rows, n_features, dtype=np.float32, nan_frac=0.1, integer=False,
                categories=None):
    """Rows with NaNs, exact integers (threshold ties), negative and fractional categories."""
    rng = np.random.default_rng(seed)
    if integer:
        X = rng.integers(-3, 4, size=(n_rows, n_features)).astype(dtype)
    else:
        X = rng.standard_normal((n_rows, n_features)).astype(dtype)
    if categories is not None:
        C_ = rng.integers(-2, categories + 3, size=(n_rows, n_features)).astype(dtype)
        C_ += (rng.random((n_rows, n_features)) < 0.2) * 0.5
        pick = rng.random((n_rows, n_features)) < 0.5
        X = np.where(pick, C_, X).astype(dtype)
    if nan_frac > 0:
        X[rng.random((n_rows, n_features)) < nan_frac] = np.nan
    return X


def py_find_leaf(desc: ForestDesc, t: int, row, precision="single"):
    """Pure-Python statement of one traversal, written from the semantics list, independent of
    the C oracle."""
    ft = np.float32 if precision == "single" else np.float64
    base = int(desc.tree_offsets[t])
    n = 0
    while desc.node_kind[base + n] != NODE_LEAF:
        g = base + n
        x = ft(row[desc.feature[g]])
        if math.isnan(float(x)):
            go_left = bool(desc.default_left[g])
        elif desc.node_kind[g] == NODE_CATEGORICAL:
            digits = 24 if precision == "single" else 53
            matched = False
            if not (x < 0) and not (abs(float(x)) > float(2 ** digits)):
                cat = int(float(x))
                lst = desc.cat_values[int(desc.cat_ptr[g]):int(desc.cat_ptr[g + 1])]
                matched = cat in set(int(c) for c in lst)
            right_on_match = bool(desc.cat_right[g]) if desc.cat_right is not None else True
            go_left = not (matched == right_on_match)
        else:
            thr = ft(desc.threshold[g])
            o = int(desc.op[g]) if desc.op is not None else desc.op_all
            go_left = {OP_LT: x < thr, OP_LE: x <= thr, OP_GT: x > thr, OP_GE: x >= thr}[o]
        n = int(desc.left[g] if go_left else desc.right[g])
    return n


def py_predict(desc: ForestDesc, X, precision="single"):
    """Leaf ids and raw (pre-postprocessing, summed) outputs by the pure-Python walker."""
    n = X.shape[0]
    ids = np.zeros((n, desc.n_trees), np.uint32)
    raw = np.zeros((n, desc.n_outputs), np.float64)
    ft = np.float32 if precision == "single" else np.float64
    k = desc.n_outputs
    for r in range(n):
        for t in range(desc.n_trees):
            lf = py_find_leaf(desc, t, X[r], precision)
            ids[r, t] = lf
            g = int(desc.tree_offsets[t]) + lf
            if desc.leaf_vector_len > 1:
                raw[r] += desc.leaf_value[g * k:(g + 1) * k].astype(ft)
            else:
                c = int(desc.class_id[t]) if desc.class_id is not None else t % k
                raw[r, c] += ft(desc.leaf_value[g])
    return ids, raw


def run_pack_check(pack_check, desc: ForestDesc, X, precision="single", layout="depth_first",
                   storage="auto", align_bytes=0, row_quantization=0, compact_image=0):
    """Pack `desc` with the product packer and walk the packed arrays on the host."""
    dt = np.float32 if precision == "single" else np.float64
    X = np.ascontiguousarray(X, dt)
    n = X.shape[0]
    ids = np.zeros((n, desc.n_trees), np.uint32)
    pay = np.zeros((n, desc.n_trees), np.float64)
    info = np.zeros(16, np.int64)
    cd = desc.to_c()
    opts = CCreateOpts(0 if precision == "single" else 1, LAYOUTS[layout], STORAGES[storage],
                       align_bytes, 0, 0, row_quantization, compact_image)
    rc = pack_check.pack_check(C.byref(cd), C.byref(opts), X.ctypes.data, n, X.shape[1],
                               ids.ctypes.data, pay.ctypes.data, info.ctypes.data)
    return rc, ids, pay, info


def load_golden(name):
    """(ForestDesc, X, dict of expected arrays) of a fixture written by tests/golden/make_golden.py."""
    import os

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name + ".npz")
    with np.load(path, allow_pickle=False) as z:
        d = {k: z[k] for k in z.files}
    fields = {}
    for k in ForestDesc._SCALARS:
        v = d["desc_" + k]
        fields[k] = v.item()
    for k in ForestDesc._ARRAYS:
        fields[k] = d.get("desc_" + k)
    fields["postproc"] = str(fields["postproc"])
    fields["native_precision"] = str(fields["native_precision"])
    exp = {k: v for k, v in d.items() if not k.startswith("desc_") and k != "X"}
    return ForestDesc(**fields), d["X"], exp


def xgboost_style_desc(seed, n_trees=24, n_features=9, max_depth=6, n_classes=1,
                       categorical=True):
    """Random ragged forest limited to what an XGBoost model file can say: `<` tests, listed
    categories go right, float32 thresholds and leaves, class of a tree in `class_id`."""
    d = random_forest_desc(seed, n_trees=n_trees, n_features=n_features, max_depth=max_depth,
                           n_outputs=n_classes, categorical=categorical, op=OP_LT,
                           postproc="softmax" if n_classes > 1 else "sigmoid")
    if d.cat_right is not None:
        d.cat_right = np.ones_like(d.cat_right)
    d.leaf_value = d.leaf_value.astype(np.float32).astype(np.float64)
    d.sigmoid_alpha = 1.0  # the format has no slope parameter
    return d


def lightgbm_style_desc(seed, n_trees=24, n_features=9, max_depth=6, n_classes=1,
                        categorical=True):
    """Random ragged forest limited to what a LightGBM text model can say: `<=` tests, listed
    categories go left and missing values right at categorical nodes, tree t feeds class t % k."""
    d = random_forest_desc(seed, n_trees=n_trees, n_features=n_features, max_depth=max_depth,
                           n_outputs=n_classes, categorical=categorical, op=OP_LE,
                           postproc="softmax" if n_classes > 1 else "sigmoid")
    if d.cat_right is not None:
        d.cat_right = np.zeros_like(d.cat_right)
        d.default_left = np.where(d.node_kind == NODE_CATEGORICAL, 0, d.default_left).astype(np.uint8)
    if n_classes > 1:
        d.class_id = (np.arange(d.n_trees) % n_classes).astype(np.int32)
    return d
