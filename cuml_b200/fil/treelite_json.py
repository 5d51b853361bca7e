"""Importer for the JSON dump of a Treelite model (`treelite.Model.dump_as_json()`).

The reference hands Treelite models to its inference library
(python/cuml/cuml/ensemble/randomforest_common.pyx:402-409); Treelite itself is not installed
here, so this reader consumes the model's JSON dump instead.  Field names seen in the reference's
own tests: `trees[].nodes[]` with `node_id`, `left_child`, `right_child`, `leaf_value`,
`data_count`, `node_type == "categorical_test_node"` (python/cuml/tests/test_random_forest.py:1185-1192,
python/cuml/tests/explainer/test_gpu_treeshap.py:97-107).  The remaining names follow Treelite
4.x's documented dump format.  Not validated against a real Treelite install.
"""
from __future__ import annotations

import numpy as np

from ._desc import (NODE_CATEGORICAL, NODE_LEAF, NODE_NUMERICAL, OP_GE, OP_GT, OP_LE, OP_LT,
                    ForestDesc)

_OPS = {"<": OP_LT, "<=": OP_LE, ">": OP_GT, ">=": OP_GE}


def from_treelite_json(model: dict) -> ForestDesc:
    trees = model["trees"]
    n_features = int(model["num_feature"])
    num_target = int(model.get("num_target", 1))
    if num_target != 1:
        raise ValueError("multi-target Treelite models are not supported")
    num_class = model.get("num_class", [1])
    k = int(num_class[0] if isinstance(num_class, (list, tuple)) else num_class)
    lvs = model.get("leaf_vector_shape", [1, 1])
    vec_len = int(lvs[-1]) if isinstance(lvs, (list, tuple)) else 1
    vec_len = vec_len if vec_len > 1 else 1
    kind, feat, thr, left, right, dl, op, leaf = [], [], [], [], [], [], [], []
    cat_ptr, cat_vals, cat_right = [0], [], []
    offs = [0]
    any_cat = False
    for tree in trees:
        nodes = sorted(tree["nodes"], key=lambda nd: nd["node_id"])
        id2rel = {nd["node_id"]: i for i, nd in enumerate(nodes)}
        for nd in nodes:
            cats = []
            cr = 1
            if "leaf_value" in nd:
                kind.append(NODE_LEAF)
                feat.append(0); thr.append(0.0); left.append(-1); right.append(-1)
                dl.append(0); op.append(OP_LT)
                v = nd["leaf_value"]
                v = np.asarray(v if isinstance(v, (list, tuple)) else [v], np.float64)
                if v.shape[0] != vec_len:
                    raise ValueError("leaf vector length differs from leaf_vector_shape")
                leaf.append(v)
            else:
                is_cat = nd.get("node_type") == "categorical_test_node"
                kind.append(NODE_CATEGORICAL if is_cat else NODE_NUMERICAL)
                feat.append(int(nd["split_feature_id"]))
                left.append(id2rel[nd["left_child"]])
                right.append(id2rel[nd["right_child"]])
                dl.append(1 if nd.get("default_left", False) else 0)
                leaf.append(np.zeros(vec_len))
                if is_cat:
                    any_cat = True
                    cats = [int(c) for c in nd.get("category_list", [])]
                    cr = 1 if nd.get("category_list_right_child", False) else 0
                    thr.append(0.0); op.append(OP_LT)
                else:
                    thr.append(float(nd["threshold"]))
                    op.append(_OPS[nd.get("comparison_op", "<")])
            cat_vals.extend(cats)
            cat_ptr.append(len(cat_vals))
            cat_right.append(cr)
        offs.append(len(kind))
    class_id = model.get("class_id")
    if vec_len > 1:
        class_id = None
    elif class_id is not None:
        class_id = np.asarray(class_id, np.int32)
        if (class_id < 0).any():
            class_id = None
    post = model.get("postprocessor", "identity")
    task = str(model.get("task_type", ""))
    base = model.get("base_scores")
    return ForestDesc(
        n_features=n_features, n_outputs=k, leaf_vector_len=vec_len,
        tree_offsets=np.asarray(offs, np.int64), node_kind=kind, feature=feat, threshold=thr,
        left=left, right=right, default_left=dl, leaf_value=np.concatenate(leaf), op=op,
        cat_ptr=np.asarray(cat_ptr, np.int64) if any_cat else None,
        cat_values=np.asarray(cat_vals or [0], np.uint32) if any_cat else None,
        cat_right=cat_right if any_cat else None, class_id=class_id,
        average_tree_output=bool(model.get("average_tree_output", False)),
        base_scores=None if base is None else np.asarray(base, np.float64).ravel()[:k],
        postproc=post, sigmoid_alpha=float(model.get("sigmoid_alpha", 1.0)),
        ratio_c=float(model.get("ratio_c", 1.0)),
        is_classifier=("Clf" in task) or post in ("sigmoid", "softmax", "multiclass_ova",
                                                   "identity_multiclass"),
        native_precision="double" if model.get("threshold_type", "float64") == "float64"
        else "single")


def to_treelite_json(desc: ForestDesc) -> dict:
    """Write a description in the same dump format (used for round-trip tests and as an
    interchange file)."""
    k = desc.n_outputs
    trees = []
    for t in range(desc.n_trees):
        b, e = int(desc.tree_offsets[t]), int(desc.tree_offsets[t + 1])
        nodes = []
        for g in range(b, e):
            nd = {"node_id": g - b}
            if desc.node_kind[g] == NODE_LEAF:
                w = desc.leaf_vector_len
                v = desc.leaf_value[g * w:(g + 1) * w]
                nd["leaf_value"] = float(v[0]) if w == 1 else [float(x) for x in v]
            else:
                nd["split_feature_id"] = int(desc.feature[g])
                nd["default_left"] = bool(desc.default_left[g])
                nd["left_child"] = int(desc.left[g])
                nd["right_child"] = int(desc.right[g])
                if desc.node_kind[g] == NODE_CATEGORICAL:
                    nd["node_type"] = "categorical_test_node"
                    nd["category_list"] = [int(c) for c in desc.cat_values[
                        int(desc.cat_ptr[g]):int(desc.cat_ptr[g + 1])]]
                    nd["category_list_right_child"] = bool(
                        desc.cat_right[g]) if desc.cat_right is not None else True
                else:
                    nd["node_type"] = "numerical_test_node"
                    o = int(desc.op[g]) if desc.op is not None else desc.op_all
                    nd["comparison_op"] = {v: s for s, v in _OPS.items()}[o]
                    nd["threshold"] = float(desc.threshold[g])
            nodes.append(nd)
        trees.append({"num_nodes": e - b, "nodes": nodes})
    cid = desc.class_id
    if cid is None:
        cid = ([-1] * desc.n_trees if desc.leaf_vector_len > 1
               else [t % k for t in range(desc.n_trees)])
    return {
        "num_feature": desc.n_features, "num_target": 1, "num_class": [k],
        "leaf_vector_shape": [1, desc.leaf_vector_len],
        "task_type": "kMultiClf" if (desc.is_classifier and k > 1) else (
            "kBinaryClf" if desc.is_classifier else "kRegressor"),
        "average_tree_output": bool(desc.average_tree_output),
        "target_id": [0] * desc.n_trees, "class_id": [int(c) for c in cid],
        "postprocessor": desc.postproc, "sigmoid_alpha": desc.sigmoid_alpha,
        "ratio_c": desc.ratio_c,
        "base_scores": [float(b) for b in (desc.base_scores if desc.base_scores is not None
                                           else np.zeros(k))],
        "threshold_type": "float64" if desc.native_precision == "double" else "float32",
        "trees": trees}
