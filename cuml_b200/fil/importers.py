"""Front-ends that turn fitted models into a `ForestDesc`.

`from_sklearn` reads scikit-learn's own tree arrays.  It stands where the reference calls
`treelite.sklearn.import_model` (python/cuml/cuml/ensemble/randomforest_common.pyx:266) and sets
the same ensemble metadata cuML's own exporter sets for random forests: numerical test `<=`,
averaged tree outputs, vector leaves for classifiers, postprocessor identity
(cpp/src/decisiontree/decisiontree.cuh:204-205, cpp/src/randomforest/randomforest.cu:262-279).
"""
from __future__ import annotations

import numpy as np

from ._desc import (NODE_CATEGORICAL, NODE_LEAF, NODE_NUMERICAL, OP_LE, OP_LT, ForestDesc)


def _tree_arrays(tree):
    """Flat arrays of one sklearn `Tree` (children, feature, threshold, missing direction)."""
    left = np.asarray(tree.children_left, np.int32)
    right = np.asarray(tree.children_right, np.int32)
    is_leaf = left < 0
    feature = np.where(is_leaf, 0, tree.feature).astype(np.int32)
    threshold = np.where(is_leaf, 0.0, tree.threshold).astype(np.float64)
    mgl = getattr(tree, "missing_go_to_left", None)
    default_left = (np.asarray(mgl, np.uint8) if mgl is not None
                    else np.ones(left.shape[0], np.uint8))
    kind = np.where(is_leaf, NODE_LEAF, NODE_NUMERICAL).astype(np.uint8)
    return kind, feature, threshold, left, right, default_left, is_leaf


def _collect(trees, leaf_fn, width):
    offs = [0]
    parts = {k: [] for k in ("kind", "feature", "threshold", "left", "right", "dl", "leaf")}
    for tr in trees:
        kind, feature, threshold, left, right, dl, is_leaf = _tree_arrays(tr)
        parts["kind"].append(kind)
        parts["feature"].append(feature)
        parts["threshold"].append(threshold)
        parts["left"].append(left)
        parts["right"].append(right)
        parts["dl"].append(dl)
        lv = np.asarray(leaf_fn(tr), np.float64).reshape(kind.shape[0], width)
        lv = np.where(is_leaf[:, None], lv, 0.0)
        parts["leaf"].append(lv.reshape(-1))
        offs.append(offs[-1] + kind.shape[0])
    cat = {k: np.concatenate(v) for k, v in parts.items()}
    return np.asarray(offs, np.int64), cat


def from_sklearn(model) -> ForestDesc:
    """Import a fitted scikit-learn tree ensemble.

    Supported: RandomForest / ExtraTrees classifiers and regressors, single DecisionTree
    estimators, GradientBoosting classifiers and regressors, IsolationForest (path lengths are
    not transformed; use the ensemble's raw average).
    """
    name = type(model).__name__
    n_features = int(model.n_features_in_)
    if name in ("RandomForestClassifier", "ExtraTreesClassifier", "DecisionTreeClassifier"):
        if getattr(model, "n_outputs_", 1) != 1:
            raise ValueError("multi-output classifiers are not supported")
        trees = ([e.tree_ for e in model.estimators_] if hasattr(model, "estimators_")
                 else [model.tree_])
        k = int(model.n_classes_)

        def leaf(tr):
            v = np.asarray(tr.value, np.float64)[:, 0, :]
            s = v.sum(axis=1, keepdims=True)
            return v / np.where(s == 0, 1.0, s)  # class fractions of the leaf

        offs, a = _collect(trees, leaf, k)
        return ForestDesc(
            n_features=n_features, n_outputs=k, leaf_vector_len=k, tree_offsets=offs,
            node_kind=a["kind"], feature=a["feature"], threshold=a["threshold"], left=a["left"],
            right=a["right"], default_left=a["dl"], leaf_value=a["leaf"], op_all=OP_LE,
            average_tree_output=True, postproc="identity_multiclass", is_classifier=True,
            native_precision="double")
    if name in ("RandomForestRegressor", "ExtraTreesRegressor", "DecisionTreeRegressor"):
        if getattr(model, "n_outputs_", 1) != 1:
            raise ValueError("multi-output regressors are not supported")
        trees = ([e.tree_ for e in model.estimators_] if hasattr(model, "estimators_")
                 else [model.tree_])
        offs, a = _collect(trees, lambda tr: np.asarray(tr.value)[:, 0, 0], 1)
        return ForestDesc(
            n_features=n_features, n_outputs=1, leaf_vector_len=1, tree_offsets=offs,
            node_kind=a["kind"], feature=a["feature"], threshold=a["threshold"], left=a["left"],
            right=a["right"], default_left=a["dl"], leaf_value=a["leaf"], op_all=OP_LE,
            average_tree_output=True, postproc="identity", is_classifier=False,
            native_precision="double")
    if name in ("GradientBoostingClassifier", "GradientBoostingRegressor"):
        est = model.estimators_  # (n_stages, K)
        n_stage, K = est.shape
        trees = [est[i, j].tree_ for i in range(n_stage) for j in range(K)]
        lr = float(model.learning_rate)
        offs, a = _collect(trees, lambda tr: lr * np.asarray(tr.value)[:, 0, 0], 1)
        base = np.asarray(model._raw_predict_init(np.zeros((1, n_features))), np.float64).ravel()
        is_clf = name.endswith("Classifier")
        post = "identity"
        if is_clf:
            post = "sigmoid" if K == 1 else "softmax"
        return ForestDesc(
            n_features=n_features, n_outputs=K, leaf_vector_len=1, tree_offsets=offs,
            node_kind=a["kind"], feature=a["feature"], threshold=a["threshold"], left=a["left"],
            right=a["right"], default_left=a["dl"], leaf_value=a["leaf"], op_all=OP_LE,
            class_id=(np.arange(n_stage * K) % K).astype(np.int32), average_tree_output=False,
            base_scores=base, postproc=post, is_classifier=is_clf, native_precision="double")
    if name == "IsolationForest":
        from sklearn.ensemble._iforest import _average_path_length

        trees = [e.tree_ for e in model.estimators_]
        if any(not np.array_equal(f, np.arange(n_features)) for f in model.estimators_features_):
            raise ValueError("IsolationForest with feature subsampling is not supported")

        def leaf(tr):
            # isolation depth of each node plus the expected remaining path length of its samples
            depth = np.zeros(tr.node_count)
            for i in range(tr.node_count):
                if tr.children_left[i] >= 0:
                    depth[tr.children_left[i]] = depth[i] + 1
                    depth[tr.children_right[i]] = depth[i] + 1
            return depth + _average_path_length(np.asarray(tr.n_node_samples))

        offs, a = _collect(trees, leaf, 1)
        return ForestDesc(
            n_features=n_features, n_outputs=1, leaf_vector_len=1, tree_offsets=offs,
            node_kind=a["kind"], feature=a["feature"], threshold=a["threshold"], left=a["left"],
            right=a["right"], default_left=a["dl"], leaf_value=a["leaf"], op_all=OP_LE,
            average_tree_output=True, postproc="identity", is_classifier=False,
            native_precision="double")
    raise TypeError(f"unsupported scikit-learn model: {name}")


def synthetic_complete_forest(n_trees, depth, n_features, seed, n_classes=1, n_categorical=0,
                              n_categories=32, postproc=None, op=OP_LT, leaf_sigma=0.1,
                              random_default_left=True) -> ForestDesc:
    """Seeded random gradient-boosted forest of complete binary trees in heap order.

    Every internal node draws its feature uniformly, its threshold from N(0,1) and its
    missing-value direction from Bernoulli(0.5); leaves are N(0, leaf_sigma).  The first
    `n_categorical` features are categorical: a node that splits on one lists a random non-empty
    subset of {0..n_categories-1} and sends listed categories right.  With `n_classes` > 1 tree
    t feeds class t % n_classes.
    """
    rng = np.random.default_rng(seed)
    n_int = (1 << depth) - 1
    n_nodes = (1 << (depth + 1)) - 1
    total = n_trees * n_nodes
    kind = np.zeros((n_trees, n_nodes), np.uint8)
    kind[:, :n_int] = NODE_NUMERICAL
    feature = np.zeros((n_trees, n_nodes), np.int32)
    feature[:, :n_int] = rng.integers(0, n_features, size=(n_trees, n_int), dtype=np.int32)
    threshold = np.zeros((n_trees, n_nodes), np.float64)
    threshold[:, :n_int] = rng.standard_normal((n_trees, n_int)).astype(np.float32)
    idx = np.arange(n_nodes, dtype=np.int32)
    left = np.where(idx < n_int, 2 * idx + 1, -1).astype(np.int32)
    right = np.where(idx < n_int, 2 * idx + 2, -1).astype(np.int32)
    dl = np.zeros((n_trees, n_nodes), np.uint8)
    if random_default_left:
        dl[:, :n_int] = rng.integers(0, 2, size=(n_trees, n_int), dtype=np.uint8)
    leaf = np.zeros((n_trees, n_nodes), np.float64)
    leaf[:, n_int:] = (leaf_sigma * rng.standard_normal((n_trees, n_nodes - n_int))).astype(
        np.float32)
    cat_ptr = cat_values = None
    if n_categorical > 0:
        is_cat = (feature < n_categorical) & (kind == NODE_NUMERICAL)
        kind[is_cat] = NODE_CATEGORICAL
        flat = is_cat.reshape(-1)
        n_cat_nodes = int(flat.sum())
        masks = rng.integers(0, 2, size=(n_cat_nodes, n_categories), dtype=np.uint8)
        empty = masks.sum(axis=1) == 0
        masks[empty, rng.integers(0, n_categories, size=int(empty.sum()))] = 1
        counts = np.zeros(total, np.int64)
        counts[flat] = masks.sum(axis=1)
        cat_ptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        cat_values = np.nonzero(masks)[1].astype(np.uint32)
        threshold[is_cat] = 0.0
    if postproc is None:
        postproc = "sigmoid" if n_classes == 1 else "softmax"
    return ForestDesc(
        n_features=n_features, n_outputs=n_classes, leaf_vector_len=1,
        tree_offsets=np.arange(n_trees + 1, dtype=np.int64) * n_nodes,
        node_kind=kind.reshape(-1), feature=feature.reshape(-1), threshold=threshold.reshape(-1),
        left=np.tile(left, n_trees), right=np.tile(right, n_trees),
        default_left=dl.reshape(-1), leaf_value=leaf.reshape(-1), op_all=op,
        cat_ptr=cat_ptr, cat_values=cat_values,
        class_id=(np.arange(n_trees) % n_classes).astype(np.int32) if n_classes > 1 else None,
        average_tree_output=False, postproc=postproc, is_classifier=True,
        native_precision="single")
