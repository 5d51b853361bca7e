"""Importer for XGBoost's JSON model file (`Booster.save_model("model.json")`).

XGBoost tests `x < split_condition` (true goes left), sends missing values where `default_left`
says, and for categorical splits sends the listed categories right.  Leaf values live in
`split_conditions` of leaf nodes.  Written from the published schema of the format; XGBoost is not
installed here, so it has only been exercised on files produced by this library's own tests.
"""
from __future__ import annotations

import math

import numpy as np

from ._desc import NODE_CATEGORICAL, NODE_LEAF, NODE_NUMERICAL, OP_LT, ForestDesc


def from_xgboost_json(model: dict) -> ForestDesc:
    learner = model["learner"]
    gb = learner["gradient_booster"]
    if "model" not in gb:
        raise ValueError("only tree boosters (gbtree / dart without weights) are supported")
    if gb.get("name") == "dart":
        raise ValueError("dart boosters are not supported")
    gbm = gb["model"]
    lmp = learner["learner_model_param"]
    n_features = int(lmp["num_feature"])
    num_class = max(1, int(lmp.get("num_class", "0")))
    objective = learner["objective"]["name"]
    base_score = float(lmp.get("base_score", "0.5").strip("[]").split(",")[0])
    kind, feat, thr, left, right, dl, leaf = [], [], [], [], [], [], []
    cat_ptr, cat_vals = [0], []
    offs = [0]
    any_cat = False
    for tree in gbm["trees"]:
        lc, rc = tree["left_children"], tree["right_children"]
        si, sc, dfl = tree["split_indices"], tree["split_conditions"], tree["default_left"]
        st = tree.get("split_type", [0] * len(lc))
        cat_nodes = {int(n): i for i, n in enumerate(tree.get("categories_nodes", []))}
        seg, siz = tree.get("categories_segments", []), tree.get("categories_sizes", [])
        cats = tree.get("categories", [])
        for i in range(len(lc)):
            mine = []
            if lc[i] == -1:
                kind.append(NODE_LEAF)
                feat.append(0); thr.append(0.0); left.append(-1); right.append(-1); dl.append(0)
                leaf.append(float(sc[i]))
            else:
                is_cat = int(st[i]) == 1
                kind.append(NODE_CATEGORICAL if is_cat else NODE_NUMERICAL)
                feat.append(int(si[i])); left.append(int(lc[i])); right.append(int(rc[i]))
                dl.append(1 if dfl[i] else 0)
                leaf.append(0.0)
                if is_cat:
                    any_cat = True
                    j = cat_nodes[i]
                    mine = [int(c) for c in cats[int(seg[j]):int(seg[j]) + int(siz[j])]]
                    thr.append(0.0)
                else:
                    thr.append(float(sc[i]))
            cat_vals.extend(mine)
            cat_ptr.append(len(cat_vals))
        offs.append(len(kind))
    tree_info = [int(c) for c in gbm.get("tree_info", [0] * (len(offs) - 1))]
    post, base, is_clf, k = "identity", base_score, False, 1
    if objective in ("binary:logistic", "reg:logistic"):
        post, is_clf = "sigmoid", objective == "binary:logistic"
        base = math.log(base_score / (1.0 - base_score))
    elif objective == "binary:logitraw":
        is_clf = True
        base = math.log(base_score / (1.0 - base_score))
    elif objective in ("multi:softprob", "multi:softmax"):
        post, is_clf, k = "softmax", True, num_class
    elif objective in ("count:poisson", "reg:gamma", "reg:tweedie", "survival:cox"):
        post = "exponential"
        base = math.log(base_score)
    elif objective == "binary:hinge":
        post, is_clf = "hinge", True
    return ForestDesc(
        n_features=n_features, n_outputs=k, leaf_vector_len=1,
        tree_offsets=np.asarray(offs, np.int64), node_kind=kind, feature=feat, threshold=thr,
        left=left, right=right, default_left=dl, leaf_value=leaf, op_all=OP_LT,
        cat_ptr=np.asarray(cat_ptr, np.int64) if any_cat else None,
        cat_values=np.asarray(cat_vals or [0], np.uint32) if any_cat else None,
        cat_right=None, class_id=np.asarray(tree_info, np.int32) if k > 1 else None,
        average_tree_output=False, base_scores=np.full(k, base), postproc=post,
        is_classifier=is_clf, native_precision="single")


def to_xgboost_json(desc: ForestDesc, objective: str = "reg:squarederror") -> dict:
    """Write a forest description in the schema `from_xgboost_json` reads (test files and
    round trips; XGBoost itself is not involved).  The description must use what the format can
    say: `<` tests, listed categories going right, scalar leaves, no averaging."""
    if desc.leaf_vector_len != 1 or desc.average_tree_output:
        raise ValueError("the XGBoost schema holds scalar leaves and summed trees only")
    if desc.op is not None and np.any(np.asarray(desc.op)[np.asarray(desc.node_kind) == NODE_NUMERICAL] != OP_LT):
        raise ValueError("the XGBoost schema tests x < threshold only")
    if desc.op is None and desc.op_all != OP_LT and np.any(np.asarray(desc.node_kind) == NODE_NUMERICAL):
        raise ValueError("the XGBoost schema tests x < threshold only")
    if desc.cat_right is not None and np.any(
            np.asarray(desc.cat_right)[np.asarray(desc.node_kind) == NODE_CATEGORICAL] == 0):
        raise ValueError("in the XGBoost schema listed categories go right")
    trees = []
    offs = np.asarray(desc.tree_offsets)
    for t in range(desc.n_trees):
        b, e = int(offs[t]), int(offs[t + 1])
        lc, rc, si, sc, dfl, st = [], [], [], [], [], []
        cats, cnodes, csegs, csizes = [], [], [], []
        for g in range(b, e):
            k = int(desc.node_kind[g])
            if k == NODE_LEAF:
                lc.append(-1); rc.append(-1); si.append(0); dfl.append(0); st.append(0)
                sc.append(float(desc.leaf_value[g]))
                continue
            lc.append(int(desc.left[g])); rc.append(int(desc.right[g]))
            si.append(int(desc.feature[g])); dfl.append(int(desc.default_left[g]))
            if k == NODE_CATEGORICAL:
                st.append(1); sc.append(0.0)
                mine = [int(c) for c in desc.cat_values[int(desc.cat_ptr[g]):int(desc.cat_ptr[g + 1])]]
                cnodes.append(g - b); csegs.append(len(cats)); csizes.append(len(mine))
                cats.extend(mine)
            else:
                st.append(0); sc.append(float(desc.threshold[g]))
        trees.append({"left_children": lc, "right_children": rc, "split_indices": si,
                      "split_conditions": sc, "default_left": dfl, "split_type": st,
                      "categories": cats, "categories_nodes": cnodes,
                      "categories_segments": csegs, "categories_sizes": csizes,
                      "tree_param": {"num_nodes": str(e - b)}})
    k = desc.n_outputs
    info = ([int(c) for c in desc.class_id] if desc.class_id is not None
            else [t % k for t in range(desc.n_trees)])
    return {"learner": {"learner_model_param": {"num_feature": str(desc.n_features),
                                                "num_class": str(k if k > 1 else 0),
                                                "base_score": "5E-1" if objective.startswith("binary") else "0E0"},
                        "objective": {"name": objective},
                        "gradient_booster": {"name": "gbtree",
                                             "model": {"trees": trees, "tree_info": info}}},
            "version": [2, 0, 0]}
