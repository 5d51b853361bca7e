"""Importer for LightGBM's text model file (`Booster.save_model("model.txt")`).

LightGBM tests `x <= threshold` (true goes left); `decision_type` bit 0 marks a categorical split
(listed categories go LEFT), bit 1 the default-left flag, bits 2-3 the missing type (0 none,
1 zero, 2 NaN).  With missing type "none" LightGBM treats NaN as 0.0, which is expressed here as a
per-node default direction; missing type "zero" (zeros are missing) cannot be expressed and is
rejected.  Written from the published format; LightGBM is not installed here, so it has only been
exercised on files produced by this library's own tests.
"""
from __future__ import annotations

import numpy as np

from ._desc import NODE_CATEGORICAL, NODE_LEAF, NODE_NUMERICAL, OP_LE, ForestDesc


def _parse_blocks(text: str):
    header, trees, cur = {}, [], None
    for line in text.splitlines():
        line = line.strip()
        if line.startswith("Tree="):
            cur = {}
            trees.append(cur)
            continue
        if line.startswith("end of trees"):
            cur = None
            break
        if "=" in line:
            k, v = line.split("=", 1)
            (cur if cur is not None else header)[k] = v
    return header, trees


def from_lightgbm_text(text: str) -> ForestDesc:
    header, trees = _parse_blocks(text)
    n_features = int(header["max_feature_idx"]) + 1
    num_class = int(header.get("num_class", "1"))
    per_iter = int(header.get("num_tree_per_iteration", str(num_class)))
    objective = header.get("objective", "regression").split()
    kind, feat, thr, left, right, dl, leaf = [], [], [], [], [], [], []
    cat_ptr, cat_vals, cat_right = [0], [], []
    offs = [0]
    any_cat = False
    for tr in trees:
        n_leaves = int(tr["num_leaves"])
        leaf_vals = [float(x) for x in tr["leaf_value"].split()]
        if n_leaves == 1:
            kind.append(NODE_LEAF); feat.append(0); thr.append(0.0); left.append(-1)
            right.append(-1); dl.append(0); leaf.append(leaf_vals[0])
            cat_ptr.append(len(cat_vals)); cat_right.append(1)
            offs.append(len(kind))
            continue
        sf = [int(x) for x in tr["split_feature"].split()]
        th = [float(x) for x in tr["threshold"].split()]
        dt = [int(x) for x in tr["decision_type"].split()]
        lch = [int(x) for x in tr["left_child"].split()]
        rch = [int(x) for x in tr["right_child"].split()]
        cb = [int(x) for x in tr.get("cat_boundaries", "").split()]
        ct = [int(x) for x in tr.get("cat_threshold", "").split()]
        n_int = n_leaves - 1

        def rel(c):  # internal nodes first, then leaves; a negative child c names leaf ~c
            return c if c >= 0 else n_int + (~c)

        for i in range(n_int):
            is_cat = dt[i] & 1
            default_left = (dt[i] >> 1) & 1
            missing = (dt[i] >> 2) & 3
            mine = []
            if missing == 1:
                raise ValueError("LightGBM missing type 'zero' is not supported")
            feat.append(sf[i]); left.append(rel(lch[i])); right.append(rel(rch[i]))
            leaf.append(0.0)
            if is_cat:
                any_cat = True
                kind.append(NODE_CATEGORICAL)
                j = int(th[i])
                words = ct[cb[j]:cb[j + 1]]
                mine = [w * 32 + b for w, word in enumerate(words) for b in range(32)
                        if (word >> b) & 1]
                thr.append(0.0)
                cat_right.append(0)  # listed categories go left
                dl.append(0)         # NaN is not a listed category: right
            else:
                kind.append(NODE_NUMERICAL)
                thr.append(th[i])
                cat_right.append(1)
                dl.append(default_left if missing == 2 else (1 if 0.0 <= th[i] else 0))
            cat_vals.extend(mine)
            cat_ptr.append(len(cat_vals))
        for v in leaf_vals:
            kind.append(NODE_LEAF); feat.append(0); thr.append(0.0); left.append(-1)
            right.append(-1); dl.append(0); leaf.append(v)
            cat_ptr.append(len(cat_vals)); cat_right.append(1)
        offs.append(len(kind))
    n_trees = len(offs) - 1
    post, is_clf, k = "identity", False, 1
    alpha = 1.0
    if objective[0] == "binary":
        post, is_clf = "sigmoid", True
        for tok in objective[1:]:
            if tok.startswith("sigmoid:"):
                alpha = float(tok.split(":")[1])
    elif objective[0] in ("multiclass", "softmax"):
        post, is_clf, k = "softmax", True, num_class
    elif objective[0] == "multiclassova":
        post, is_clf, k = "multiclass_ova", True, num_class
        for tok in objective[1:]:
            if tok.startswith("sigmoid:"):
                alpha = float(tok.split(":")[1])
    elif objective[0] in ("poisson", "gamma", "tweedie"):
        post = "exponential"
    average = "average_output" in header or any(
        ln.strip() == "average_output" for ln in text.splitlines()[:40])
    return ForestDesc(
        n_features=n_features, n_outputs=k, leaf_vector_len=1,
        tree_offsets=np.asarray(offs, np.int64), node_kind=kind, feature=feat, threshold=thr,
        left=left, right=right, default_left=dl, leaf_value=leaf, op_all=OP_LE,
        cat_ptr=np.asarray(cat_ptr, np.int64) if any_cat else None,
        cat_values=np.asarray(cat_vals or [0], np.uint32) if any_cat else None,
        cat_right=cat_right if any_cat else None,
        class_id=(np.arange(n_trees) % per_iter).astype(np.int32) if k > 1 else None,
        average_tree_output=bool(average), postproc=post, sigmoid_alpha=alpha,
        is_classifier=is_clf, native_precision="double")


def to_lightgbm_text(desc: ForestDesc, objective: str = "regression") -> str:
    """Write a forest description in the text format `from_lightgbm_text` reads (test files and
    round trips; LightGBM itself is not involved).  The description must use what the format can
    say: `<=` tests, listed categories going left with missing values going right at categorical
    nodes, scalar leaves, tree t feeding class t % n_classes.  Internal nodes are renumbered
    first and leaves after them, as the format prescribes, so leaf ids change."""
    kinds = np.asarray(desc.node_kind)
    if desc.leaf_vector_len != 1:
        raise ValueError("the LightGBM format holds scalar leaves only")
    ops = np.asarray(desc.op) if desc.op is not None else np.full(len(kinds), desc.op_all)
    if np.any(ops[kinds == NODE_NUMERICAL] != OP_LE):
        raise ValueError("the LightGBM format tests x <= threshold only")
    if np.any(kinds == NODE_CATEGORICAL):
        cr = np.asarray(desc.cat_right) if desc.cat_right is not None else np.ones(len(kinds))
        if np.any(cr[kinds == NODE_CATEGORICAL] != 0) or np.any(
                np.asarray(desc.default_left)[kinds == NODE_CATEGORICAL] != 0):
            raise ValueError("LightGBM categorical tests send listed categories left and "
                             "missing values right")
    k = desc.n_outputs
    if k > 1 and desc.class_id is not None and np.any(
            np.asarray(desc.class_id) != np.arange(desc.n_trees) % k):
        raise ValueError("LightGBM trees feed class t % n_classes")
    lines = ["tree", "version=v3", f"num_class={k}", f"num_tree_per_iteration={k}",
             "label_index=0", f"max_feature_idx={desc.n_features - 1}", f"objective={objective}",
             ""]
    if desc.average_tree_output:
        lines.insert(7, "average_output")
    offs = np.asarray(desc.tree_offsets)

    def fmt(v):
        return repr(float(v))

    for t in range(desc.n_trees):
        b, e = int(offs[t]), int(offs[t + 1])
        internal = [g for g in range(b, e) if kinds[g] != NODE_LEAF]
        leaves = [g for g in range(b, e) if kinds[g] == NODE_LEAF]
        ipos = {g: i for i, g in enumerate(internal)}
        lpos = {g: i for i, g in enumerate(leaves)}
        if kinds[b] != NODE_LEAF and ipos[b] != 0:
            raise ValueError("the root must be the tree's first node")

        def child(rel):
            g = b + int(rel)
            return ipos[g] if g in ipos else ~lpos[g]

        lines.append(f"Tree={t}")
        lines.append(f"num_leaves={len(leaves)}")
        sf, th, dt, lch, rch, cb, ct = [], [], [], [], [], [0], []
        for g in internal:
            sf.append(int(desc.feature[g]))
            lch.append(child(desc.left[g])); rch.append(child(desc.right[g]))
            if kinds[g] == NODE_CATEGORICAL:
                mine = [int(c) for c in desc.cat_values[int(desc.cat_ptr[g]):int(desc.cat_ptr[g + 1])]]
                n_words = (max(mine) // 32 + 1) if mine else 1
                words = [0] * n_words
                for c in mine:
                    words[c // 32] |= 1 << (c % 32)
                th.append(float(len(cb) - 1))
                ct.extend(words); cb.append(len(ct))
                dt.append(1 | (2 << 2))
            else:
                th.append(float(desc.threshold[g]))
                dt.append((int(desc.default_left[g]) << 1) | (2 << 2))  # missing type NaN
        lines.append(f"num_cat={len(cb) - 1}")
        if internal:
            lines.append("split_feature=" + " ".join(map(str, sf)))
            lines.append("threshold=" + " ".join(fmt(v) for v in th))
            lines.append("decision_type=" + " ".join(map(str, dt)))
            lines.append("left_child=" + " ".join(map(str, lch)))
            lines.append("right_child=" + " ".join(map(str, rch)))
        lines.append("leaf_value=" + " ".join(fmt(desc.leaf_value[g]) for g in leaves))
        if len(cb) > 1:
            lines.append("cat_boundaries=" + " ".join(map(str, cb)))
            lines.append("cat_threshold=" + " ".join(map(str, ct)))
        lines.append("shrinkage=1")
        lines.append("")
    lines.append("end of trees")
    lines.append("")
    return "\n".join(lines)
