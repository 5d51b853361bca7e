"""The CPU oracle against (a) scikit-learn's own outputs stored in tests/golden/ and (b) a
pure-Python walker written from the semantics list, on tiny forests covering operators,
categorical lists, missing values, vector leaves and every postprocessor."""
import numpy as np
import pytest

from cuml_b200.fil._desc import (INFER_CLASS, INFER_DEFAULT, INFER_LEAF_ID, INFER_PER_TREE,
                                 INFER_PROBA2, OP_GE, OP_GT, OP_LE, OP_LT)
from oracle import oracle
from tests.helpers import load_golden, py_predict, random_forest_desc, random_rows


def test_golden_rfc_depth8():
    desc, X, exp = load_golden("rfc_depth8")
    for prec in ("single", "double"):
        ids = oracle.predict(desc, X, INFER_LEAF_ID, prec)
        assert np.array_equal(ids.astype(np.int64), exp["leaf_ids"])
        proba = oracle.predict(desc, X, INFER_DEFAULT, prec)
        np.testing.assert_allclose(proba, exp["proba"], rtol=1e-6, atol=1e-7)
        cls = oracle.predict(desc, X, INFER_CLASS, prec)
        assert np.array_equal(cls.astype(np.int64), exp["labels"])


def test_golden_rfr_depth20_fp64():
    desc, X, exp = load_golden("rfr_depth20")
    ids = oracle.predict(desc, X, INFER_LEAF_ID, "double")
    assert np.array_equal(ids.astype(np.int64), exp["leaf_ids"])
    vals = oracle.predict(desc, X, INFER_DEFAULT, "double")
    np.testing.assert_allclose(vals[:, 0], exp["values"], rtol=1e-12, atol=1e-12)


def test_golden_gbc_3class():
    desc, X, exp = load_golden("gbc_3class")
    proba = oracle.predict(desc, X, INFER_DEFAULT, "double")
    np.testing.assert_allclose(proba, exp["proba"], rtol=1e-12, atol=1e-14)
    cls = oracle.predict(desc, X, INFER_CLASS, "double")
    assert np.array_equal(cls.astype(np.int64), exp["labels"])


def test_golden_missing_values():
    desc, X, exp = load_golden("rfc_missing")
    assert np.isnan(X).any()
    ids = oracle.predict(desc, X, INFER_LEAF_ID, "single")
    assert np.array_equal(ids.astype(np.int64), exp["leaf_ids"])
    proba = oracle.predict(desc, X, INFER_DEFAULT, "single")
    np.testing.assert_allclose(proba, exp["proba"], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("op", [OP_LT, OP_LE, OP_GT, OP_GE])
@pytest.mark.parametrize("precision", ["single", "double"])
def test_operators_and_ties_vs_python(op, precision):
    # integer thresholds and integer inputs force x == threshold ties, where < and <= differ
    desc = random_forest_desc(10 + op, n_trees=5, max_depth=4, op=op, integer_thresholds=True)
    X = random_rows(1, 200, desc.n_features, np.float64, nan_frac=0.1, integer=True)
    ids_py, raw_py = py_predict(desc, X, precision)
    ids = oracle.predict(desc, X, INFER_LEAF_ID, precision)
    assert np.array_equal(ids, ids_py)
    out = oracle.predict(desc, X, INFER_DEFAULT, precision)
    np.testing.assert_allclose(out, raw_py, rtol=1e-6 if precision == "single" else 1e-12, atol=1e-6)


@pytest.mark.parametrize("big", [False, True])
def test_categorical_vs_python(big):
    desc = random_forest_desc(20 + big, n_trees=8, max_depth=5, categorical=True,
                              big_categories=big, mixed_ops=True)
    X = random_rows(2, 300, desc.n_features, np.float32, nan_frac=0.1, categories=75 if big else 22)
    ids_py, _ = py_predict(desc, X, "single")
    ids = oracle.predict(desc, X, INFER_LEAF_ID, "single")
    assert np.array_equal(ids, ids_py)


def test_vector_leaves_and_per_tree():
    desc = random_forest_desc(30, n_trees=6, n_outputs=4, vector=True, average=True)
    X = random_rows(3, 100, desc.n_features, np.float32)
    ids_py, raw_py = py_predict(desc, X, "single")
    out = oracle.predict(desc, X, INFER_DEFAULT, "single")
    np.testing.assert_allclose(out, raw_py / desc.n_trees, rtol=1e-6, atol=1e-7)
    pt = oracle.predict(desc, X, INFER_PER_TREE, "single")
    assert pt.shape == (100, 6, 4)
    np.testing.assert_allclose(pt.sum(axis=1) / 6, out, rtol=1e-5, atol=1e-6)
    cls = oracle.predict(desc, X, INFER_CLASS, "single")
    assert np.array_equal(cls, np.argmax(out, axis=1))


def test_multiclass_scalar_leaves_average_per_class():
    desc = random_forest_desc(31, n_trees=9, n_outputs=3, average=True, base=True)
    X = random_rows(4, 100, desc.n_features, np.float64)
    _, raw_py = py_predict(desc, X, "double")
    counts = np.bincount(desc.class_id, minlength=3).astype(np.float64)
    want = raw_py / np.where(counts == 0, 1, counts) + desc.base_scores
    out = oracle.predict(desc, X, INFER_DEFAULT, "double")
    np.testing.assert_allclose(out, want, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("post", ["sigmoid", "exponential", "logarithm_one_plus_exp",
                                  "signed_square", "hinge", "softmax", "multiclass_ova",
                                  "exponential_standard_ratio"])
def test_postprocessors(post):
    k = 3 if post in ("softmax", "multiclass_ova") else 1
    desc = random_forest_desc(40, n_trees=6, n_outputs=k, postproc=post)
    X = random_rows(5, 64, desc.n_features, np.float64, nan_frac=0.0)
    _, s = py_predict(desc, X, "double")
    a = desc.sigmoid_alpha
    want = {
        "sigmoid": lambda: 1 / (1 + np.exp(-a * s)),
        "multiclass_ova": lambda: 1 / (1 + np.exp(-a * s)),
        "exponential": lambda: np.exp(s),
        "logarithm_one_plus_exp": lambda: np.log1p(np.exp(s)),
        "signed_square": lambda: np.sign(s) * s * s,
        "hinge": lambda: (s > 0).astype(np.float64),
        "softmax": lambda: np.exp(s - s.max(1, keepdims=True)) /
        np.exp(s - s.max(1, keepdims=True)).sum(1, keepdims=True),
        "exponential_standard_ratio": lambda: np.exp2(-s / desc.ratio_c),
    }[post]()
    out = oracle.predict(desc, X, INFER_DEFAULT, "double")
    np.testing.assert_allclose(out, want, rtol=1e-12, atol=1e-14)
    if post == "sigmoid":
        p2 = oracle.predict(desc, X, INFER_PROBA2, "double")
        np.testing.assert_allclose(p2[:, 1], want[:, 0], rtol=1e-12)
        np.testing.assert_allclose(p2.sum(1), 1.0, rtol=1e-12)
        cls = oracle.predict(desc, X, INFER_CLASS, "double", threshold=0.3)
        assert np.array_equal(cls, (want[:, 0] > 0.3).astype(np.int32))


def test_fp32_threshold_rounding_case():
    """A forest imported at single precision rounds fp64 thresholds to fp32; a row that equals
    the rounded threshold exactly shows the difference between the two precisions."""
    t64 = 0.1  # not representable in fp32; float32(0.1) > 0.1
    desc = random_forest_desc(0, n_trees=1, max_depth=0)
    from cuml_b200.fil._desc import ForestDesc, NODE_LEAF, NODE_NUMERICAL

    desc = ForestDesc(n_features=1, n_outputs=1, tree_offsets=[0, 3],
                      node_kind=[NODE_NUMERICAL, NODE_LEAF, NODE_LEAF], feature=[0, 0, 0],
                      threshold=[t64, 0, 0], left=[1, -1, -1], right=[2, -1, -1],
                      default_left=[1, 0, 0], leaf_value=[0, 1.0, 2.0], op_all=OP_LE)
    x = np.array([[np.float32(t64)]], np.float64)  # fl32(t64), slightly above t64
    assert oracle.predict(desc, x, INFER_LEAF_ID, "double")[0, 0] == 2  # x > t64
    assert oracle.predict(desc, x, INFER_LEAF_ID, "single")[0, 0] == 1  # x <= fl32(t64)


def test_empty_batch_and_single_leaf_tree():
    desc = random_forest_desc(50, n_trees=3, max_depth=0)  # every tree is one leaf
    X = np.zeros((0, desc.n_features), np.float32)
    assert oracle.predict(desc, X, INFER_DEFAULT, "single").shape == (0, 1)
    X = np.zeros((2, desc.n_features), np.float32)
    ids = oracle.predict(desc, X, INFER_LEAF_ID, "single")
    assert np.array_equal(ids, np.zeros((2, 3), np.uint32))


def test_packed_walk_equals_plain_walk():
    """The packed walk (one record per node, eight rows side by side) is what the benchmarks time
    as the CPU baseline; it must give exactly what the plain walk gives, for every output kind."""
    from cuml_b200.fil._desc import (INFER_CLASS, INFER_DEFAULT, INFER_LEAF_ID, INFER_PER_TREE,
                                     INFER_PROBA2)
    from tests.helpers import load_golden, random_forest_desc, random_rows

    cases = [
        (random_forest_desc(1, n_trees=15, max_depth=7, mixed_ops=True, integer_thresholds=True,
                            postproc="sigmoid"), dict(integer=True, nan_frac=0.15)),
        (random_forest_desc(2, n_trees=9, n_outputs=3, vector=True, average=True), dict()),
        (random_forest_desc(3, n_trees=12, n_outputs=4, postproc="softmax", base=True), dict()),
        (random_forest_desc(4, n_trees=8, categorical=True), dict(categories=22)),  # plain fallback
    ]
    for desc, kw in cases:
        X = random_rows(7, 203, desc.n_features, np.float64, **kw)  # 203: ragged last group of rows
        for precision in ("single", "double"):
            kinds = [INFER_DEFAULT, INFER_LEAF_ID, INFER_PER_TREE, INFER_CLASS]
            if desc.n_outputs == 1:
                kinds.append(INFER_PROBA2)
            for kind in kinds:
                a = oracle.predict(desc, X, kind, precision)
                b = oracle.predict(desc, X, kind, precision, packed=True)
                assert np.array_equal(a, b, equal_nan=True)
    desc, X, exp = load_golden("rfr_depth20")
    assert np.array_equal(oracle.predict(desc, X, INFER_LEAF_ID, "double", packed=True).astype(np.int64),
                          exp["leaf_ids"])
