"""The product packer (cuml_b200/csrc/pack.cpp) checked on the CPU: a test-only host walker follows
the PACKED node arrays with the kernels' index arithmetic and must reach the leaves the oracle
reaches, for every storage, node order, precision and operator normalisation."""
import ctypes as C

import numpy as np
import pytest

from cuml_b200.fil._desc import INFER_LEAF_ID, INFER_PER_TREE, OP_GE, OP_GT, OP_LE, OP_LT
from cuml_b200.fil.importers import synthetic_complete_forest
from oracle import oracle
from tests.helpers import load_golden, random_forest_desc, random_rows, run_pack_check

LAYOUT_STORAGE = [("depth_first", "sparse"), ("breadth_first", "sparse"), ("layered", "sparse"),
                  ("depth_first", "dense"), ("depth_first", "auto")]


def _check(pack_check, desc, X, precision, layout, storage, align=0):
    rc, ids, pay, info = run_pack_check(pack_check, desc, X, precision, layout, storage, align)
    assert rc == 0, pack_check.pack_check_error()
    want = oracle.predict(desc, X, INFER_LEAF_ID, precision)
    assert np.array_equal(ids, want)
    # dense forests without categorical tests also carry a rank-quantised copy; the walk over it
    # must reach exactly the same leaves
    if info[1] == 1 and desc.cat_ptr is None:
        assert info[6] == 1
    assert info[7] == 0
    # sparse forests whose fields fit also carry the compact image (internal nodes only, heap of
    # the top levels); the walk over it must reach the same leaves and payloads
    if info[1] == 2 and desc.n_features <= 4096:
        assert info[12] == 1 and info[14] >= 1
    assert info[13] == 0
    if desc.leaf_vector_len == 1:
        pt = oracle.predict(desc, X, INFER_PER_TREE, precision)
        assert np.array_equal(pay.astype(pt.dtype), pt)
    return info


@pytest.mark.parametrize("layout,storage", LAYOUT_STORAGE)
@pytest.mark.parametrize("precision", ["single", "double"])
def test_mixed_operators_ties_nan(pack_check, layout, storage, precision):
    desc = random_forest_desc(1, n_trees=9, max_depth=6, mixed_ops=True, integer_thresholds=True)
    X = random_rows(2, 400, desc.n_features, np.float64, nan_frac=0.15, integer=True)
    _check(pack_check, desc, X, precision, layout, storage)


@pytest.mark.parametrize("layout,storage", LAYOUT_STORAGE)
@pytest.mark.parametrize("big", [False, True])
def test_categorical(pack_check, layout, storage, big):
    desc = random_forest_desc(3 + big, n_trees=8, max_depth=5, categorical=True,
                              big_categories=big, mixed_ops=True)
    X = random_rows(4, 500, desc.n_features, np.float32, nan_frac=0.1, categories=75 if big else 22)
    _check(pack_check, desc, X, "single", layout, storage)
    _check(pack_check, desc, X, "double", layout, storage)


@pytest.mark.parametrize("layout,storage", LAYOUT_STORAGE)
def test_vector_leaves(pack_check, layout, storage):
    desc = random_forest_desc(5, n_trees=6, n_outputs=3, vector=True)
    X = random_rows(6, 200, desc.n_features, np.float32)
    _check(pack_check, desc, X, "single", layout, storage)


@pytest.mark.parametrize("layout,storage", LAYOUT_STORAGE)
def test_multiclass_tree_reordering_keeps_tree_index(pack_check, layout, storage):
    # scalar-leaf multi-class forests are stored class by class; ids must still be reported
    # under the tree's original index
    desc = random_forest_desc(7, n_trees=11, n_outputs=4)
    X = random_rows(8, 200, desc.n_features, np.float32)
    _check(pack_check, desc, X, "single", layout, storage)


@pytest.mark.parametrize("op", [OP_LT, OP_LE])
def test_complete_forest_dense(pack_check, op):
    desc = synthetic_complete_forest(20, 6, 16, seed=2, op=op, n_categorical=3, n_categories=32,
                                     n_classes=3)
    X = random_rows(9, 500, 16, np.float32, nan_frac=0.05, categories=32)
    info = _check(pack_check, desc, X, "single", "depth_first", "auto")
    assert info[1] == 1 and info[2] == 6  # dense storage, depth 6
    assert info[4] == 20 * 2 * 64
    # categorical features with small category sets keep the rank-quantised copy: the code of a
    # categorical value is its category (rows hold negative, fractional and too-large categories)
    assert info[6] == 1


def test_golden_forests_all_layouts(pack_check):
    for name, prec in (("rfc_depth8", "single"), ("rfr_depth20", "double"),
                       ("rfc_missing", "single")):
        desc, X, exp = load_golden(name)
        X = X[:300]
        for layout, storage in LAYOUT_STORAGE:
            if storage == "dense" and name == "rfr_depth20":
                continue  # depth 20 cannot be padded
            rc, ids, _, info = run_pack_check(pack_check, desc, X, prec, layout, storage)
            assert rc == 0, pack_check.pack_check_error()
            assert np.array_equal(ids.astype(np.int64), exp["leaf_ids"][:300])
        if name == "rfr_depth20":
            rc, _, _, info = run_pack_check(pack_check, desc, X[:1], prec, "depth_first", "auto")
            assert info[1] == 2  # AUTO falls back to sparse storage for deep ragged trees


def test_align_bytes_and_wide_nodes(pack_check):
    desc = random_forest_desc(11, n_trees=5, max_depth=7, p_leaf=0.1)
    X = random_rows(12, 100, desc.n_features, np.float32)
    info = _check(pack_check, desc, X, "single", "depth_first", "sparse", align=128)
    assert info[0] == 2 and info[3] == 8  # compact 8-byte nodes
    # many features leave too few offset bits for the compact node: the wide node is chosen
    desc = random_forest_desc(13, n_trees=3, n_features=1 << 22, max_depth=9, p_leaf=0.05)
    X = np.zeros((4, 1 << 22), np.float32)
    X[:, ::7] = 1.5
    info = _check(pack_check, desc, X, "single", "depth_first", "sparse")
    assert info[0] == 3 and info[3] == 16


def test_le_with_infinite_threshold(pack_check):
    from cuml_b200.fil._desc import ForestDesc, NODE_LEAF, NODE_NUMERICAL

    for op in (OP_LE, OP_GT, OP_LT, OP_GE):
        for thr in (np.inf, -np.inf, np.float64(np.finfo(np.float32).max), 0.0, -0.0):
            desc = ForestDesc(n_features=1, n_outputs=1, tree_offsets=[0, 3],
                              node_kind=[NODE_NUMERICAL, NODE_LEAF, NODE_LEAF], feature=[0, 0, 0],
                              threshold=[thr, 0, 0], left=[1, -1, -1], right=[2, -1, -1],
                              default_left=[0, 0, 0], leaf_value=[0, 1.0, 2.0], op_all=op)
            X = np.array([[np.inf], [-np.inf], [0.0], [-0.0], [np.nan], [3e38], [-3e38],
                          [1e-45], [-1e-45]], np.float32)
            for storage in ("sparse", "dense"):
                _check(pack_check, desc, X, "single", "depth_first", storage)
                _check(pack_check, desc, X, "double", "depth_first", storage)


def _bad(desc_kwargs):
    from cuml_b200.fil._desc import ForestDesc, NODE_LEAF, NODE_NUMERICAL

    base = dict(n_features=2, n_outputs=1, tree_offsets=[0, 3],
                node_kind=[NODE_NUMERICAL, NODE_LEAF, NODE_LEAF], feature=[0, 0, 0],
                threshold=[0.5, 0, 0], left=[1, -1, -1], right=[2, -1, -1],
                default_left=[0, 0, 0], leaf_value=[0, 1.0, 2.0])
    base.update(desc_kwargs)
    return ForestDesc(**base)


@pytest.mark.parametrize("kwargs,code", [
    (dict(left=[5, -1, -1]), -2),            # child out of range
    (dict(left=[0, -1, -1]), -2),            # cycle: the root is its own child
    (dict(right=[1, -1, -1]), -2),           # both children are the same node
    (dict(feature=[2, 0, 0]), -2),           # feature >= n_features
    (dict(feature=[-1, 0, 0]), -2),
    (dict(tree_offsets=[0, 0, 3]), -2),      # empty tree
    (dict(n_outputs=0), -1),
    (dict(leaf_vector_len=3), -1),
    (dict(node_kind=[7, 0, 0]), -2),
    (dict(op_all=9), -2),
])
def test_malformed_forests_are_rejected(pack_check, kwargs, code):
    desc = _bad(kwargs)
    rc, _, _, _ = run_pack_check(pack_check, desc, np.zeros((1, 2), np.float32))
    assert rc == code
    assert pack_check.pack_check_error() != b""


def test_bad_options_are_rejected(pack_check):
    from cuml_b200.fil._desc import CCreateOpts

    desc = _bad({})
    cd = desc.to_c()
    info = np.zeros(8, np.int64)
    for opts in (CCreateOpts(5, 0, 0, 0, 0, 0, 0, 0), CCreateOpts(0, 9, 0, 0, 0, 0, 0, 0),
                 CCreateOpts(0, 0, 7, 0, 0, 0, 0, 0), CCreateOpts(0, 0, 0, 48, 0, 0, 0, 0)):
        rc = pack_check.pack_check(C.byref(cd), C.byref(opts), None, 0, 2, None, None,
                                   info.ctypes.data)
        assert rc == -1


def test_rank_quantisation_edge_values(pack_check):
    """Ranks are exact at thresholds, next to them, at infinities, zeros of both signs and
    denormals, in both precisions; rows equal to a threshold are where `<` and `<=` differ."""
    for prec, dt in (("single", np.float32), ("double", np.float64)):
        desc = random_forest_desc(21, n_trees=30, n_features=4, max_depth=6, mixed_ops=True)
        thr = desc.threshold[desc.node_kind == 1].astype(dt)
        vals = np.concatenate([thr, np.nextafter(thr, dt(np.inf)), np.nextafter(thr, dt(-np.inf)),
                               np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45,
                                         np.finfo(dt).max, np.finfo(dt).min, np.finfo(dt).tiny],
                                        dt)])
        rng = np.random.default_rng(5)
        X = rng.choice(vals, size=(3000, 4)).astype(dt)
        info = _check(pack_check, desc, X, prec, "depth_first", "dense")
        assert info[6] == 1


def test_rank_quantisation_off_and_limits(pack_check):
    desc = random_forest_desc(22, n_trees=5, max_depth=4)
    X = random_rows(1, 50, desc.n_features, np.float32)
    rc, _, _, info = run_pack_check(pack_check, desc, X, storage="dense", row_quantization=1)
    assert rc == 0 and info[6] == 0
    # a feature with one huge threshold and one tiny one, duplicates, and an unused feature
    from cuml_b200.fil._desc import ForestDesc, NODE_LEAF, NODE_NUMERICAL

    desc = ForestDesc(n_features=3, n_outputs=1, tree_offsets=[0, 7],
                      node_kind=[1, 1, 1, 0, 0, 0, 0], feature=[0, 0, 2, 0, 0, 0, 0],
                      threshold=[1e30, 1e-30, 1e-30, 0, 0, 0, 0], left=[1, 3, 5, -1, -1, -1, -1],
                      right=[2, 4, 6, -1, -1, -1, -1], default_left=[1, 0, 1, 0, 0, 0, 0],
                      leaf_value=[0, 0, 0, 1.0, 2.0, 3.0, 4.0])
    X = np.array([[1e30, 0, 1e-30], [9e29, 1, 0], [1e-30, 2, 1e-31], [np.nan, 3, np.nan],
                  [-1, np.nan, 2e-30], [np.inf, 0, -np.inf]], np.float32)
    for prec in ("single", "double"):
        info = _check(pack_check, desc, X, prec, "depth_first", "dense")
        assert info[6] == 1


def test_rank_tables_feature_groups(pack_check):
    """The rank tables are interleaved across power-of-two groups of features: 70 features make
    groups of 32, 32, 4 and 2, and the walk over the quantised copy still reaches every leaf,
    also with NaN rows and with thresholds crowded into a few buckets."""
    desc = random_forest_desc(31, n_trees=40, n_features=70, max_depth=7, mixed_ops=True)
    # crowd the thresholds of feature 0 next to each other so that its search window grows
    num = (desc.node_kind == 1) & (desc.feature == 0)
    desc.threshold[num] = 1.0 + 1e-6 * np.arange(int(num.sum()))
    X = random_rows(32, 600, 70, np.float32, nan_frac=0.05)
    X[:200, 0] = (1.0 + 1e-6 * np.arange(200)).astype(np.float32)
    for prec in ("single", "double"):
        info = _check(pack_check, desc, X, prec, "depth_first", "dense")
        assert info[6] == 1
        assert info[8] == 4 and info[11] == 32  # groups, width of the first one
        assert info[10] <= 208 * 1024


def test_rank_quantisation_threshold_limit(pack_check):
    """A feature with more distinct thresholds than a rank can number keeps the forest on the
    plain dense path."""
    from cuml_b200.fil._desc import ForestDesc

    n = 16400  # one more stump than the 16,382 thresholds a feature may have, and then some
    kind = np.tile([1, 0, 0], n)
    desc = ForestDesc(n_features=2, n_outputs=1, tree_offsets=np.arange(0, 3 * n + 1, 3),
                      node_kind=kind, feature=np.zeros(3 * n, np.int32),
                      threshold=np.repeat(np.arange(n, dtype=np.float64), 3),
                      left=np.tile([1, -1, -1], n), right=np.tile([2, -1, -1], n),
                      default_left=np.zeros(3 * n, np.int32),
                      leaf_value=np.tile([0.0, 1.0, 2.0], n))
    X = random_rows(33, 20, 2, np.float32) * 5000
    rc, ids, _, info = run_pack_check(pack_check, desc, X, storage="dense")
    assert rc == 0 and info[1] == 1 and info[6] == 0
    assert np.array_equal(ids, oracle.predict(desc, X, INFER_LEAF_ID, "single"))


@pytest.mark.parametrize("layout", ["depth_first", "breadth_first", "layered"])
def test_compact_image_of_sparse_forests(pack_check, layout):
    """The compact image on what it was made for: deep ragged trees (deeper than the heap), fp64
    thresholds that only an exact look-up can decide, single-leaf trees, vector leaves,
    categorical tests, and the option that switches it off."""
    desc = random_forest_desc(31, n_trees=12, n_features=7, max_depth=14, p_leaf=0.12,
                              mixed_ops=True)
    thr = desc.threshold[desc.node_kind == 1]
    rng = np.random.default_rng(3)
    # rows made of thresholds and their fp64 neighbours: the float bound cannot decide them
    vals = np.concatenate([thr, np.nextafter(thr, np.inf), np.nextafter(thr, -np.inf),
                           thr.astype(np.float32).astype(np.float64), [np.nan, np.inf, -np.inf]])
    X = rng.choice(vals, size=(600, 7))
    for precision in ("single", "double"):
        info = _check(pack_check, desc, X, precision, layout, "sparse")
        assert info[12] == 1 and 1 <= info[14] <= 10
        if precision == "double":
            assert info[15] > 0  # exact look-ups happened and agreed
    rc, ids, pay, info = run_pack_check(pack_check, desc, X, "double", layout, "sparse",
                                        compact_image=1)
    assert rc == 0 and info[12] == 0
    # shallower than the heap, single-leaf trees included
    tiny = random_forest_desc(32, n_trees=6, max_depth=1, p_leaf=0.6)
    _check(pack_check, tiny, random_rows(1, 50, tiny.n_features, np.float32), "single", layout,
           "sparse")
    vec = random_forest_desc(33, n_trees=7, n_outputs=3, vector=True, max_depth=12, p_leaf=0.15)
    _check(pack_check, vec, random_rows(2, 200, vec.n_features, np.float64), "double", layout,
           "sparse")
    cat = random_forest_desc(34, n_trees=8, max_depth=11, p_leaf=0.15, categorical=True,
                             big_categories=True)
    Xc = random_rows(3, 300, cat.n_features, np.float64, categories=75)
    _check(pack_check, cat, Xc, "double", layout, "sparse")
    _check(pack_check, cat, Xc, "single", layout, "sparse")


def test_heap_levels_of_the_compact_image_follow_the_row_tile(pack_check):
    """Few features: eight heap levels.  A thousand features: the row tile takes most of shared
    memory and the heaps get fewer levels, so that a CTA still holds two dozen warps.  The walk
    over the image gives the same leaves either way."""
    levels = {}
    for n_features in (24, 1000):
        desc = random_forest_desc(90, n_trees=5, n_features=n_features, max_depth=12, p_leaf=0.1)
        X = random_rows(4, 64, n_features, np.float32)
        info = _check(pack_check, desc, X, "single", "depth_first", "sparse")
        assert info[12] == 1
        levels[n_features] = int(info[14])
    assert levels[24] == 8
    assert 1 <= levels[1000] < 8
