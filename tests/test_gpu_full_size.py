"""The benchmark configurations at their real forest shapes, through the C ABI, against the CPU
oracle and scikit-learn.

The small-shape parity tests reach the same kernel variants (the launch shape depends on depth
and feature count), but not what the tree count changes: the fp32 running sum over thousands of
leaves against the 1e-5 bar, hundreds of wrap-arounds of the tree ring per row tile, node offsets
of a forest with 2e7 nodes.  Here every configuration runs with its full forest on at least
200,000 rows; a seeded sample of those rows goes through the oracle (scores within rtol 1e-5 /
atol 1e-6 in fp32 and rtol 1e-12 in fp64, leaf ids bit-exact), and where scikit-learn trained
the forest its own `apply` / `predict_proba` / `predict` are the second witness.
"""
import numpy as np
import pytest

from cuml_b200.fil import ForestInference, synthetic_complete_forest
from cuml_b200.fil._desc import INFER_DEFAULT, INFER_LEAF_ID, INFER_PROBA2
from oracle import oracle

pytestmark = pytest.mark.gpu


def _torch():
    import torch

    return torch


def test_c1_sklearn_classifier_exact_recipe():
    """RandomForestClassifier(100 trees, max_depth 8, seed 0) fit on 10,000 make_classification
    rows (32 fp32 features, 16 informative, 2 classes); 1,000,000 fresh rows (seed 1)."""
    from sklearn.datasets import make_classification
    from sklearn.ensemble import RandomForestClassifier

    X, y = make_classification(n_samples=10_000, n_features=32, n_informative=16, n_classes=2,
                               random_state=0)
    m = RandomForestClassifier(n_estimators=100, max_depth=8, random_state=0,
                               n_jobs=-1).fit(X.astype(np.float32), y)
    Xt = make_classification(n_samples=1_000_000, n_features=32, n_informative=16, n_classes=2,
                             random_state=1)[0].astype(np.float32)
    fi = ForestInference.load_from_sklearn(m)
    d = fi.describe()
    assert fi.is_classifier and d["storage"] == 1 and d["n_trees"] == 100
    torch = _torch()
    Xd = torch.as_tensor(Xt, device="cuda:0")
    proba = fi.predict_proba(Xd).cpu().numpy()
    ids = fi.apply(Xd).cpu().numpy()
    labels = fi.predict(Xd).cpu().numpy()
    # scikit-learn itself on every row
    assert np.array_equal(ids.astype(np.int64), m.apply(Xt))
    sk = m.predict_proba(Xt)
    np.testing.assert_allclose(proba, sk, rtol=1e-5, atol=1e-6)
    safe = np.abs(sk[:, 0] - 0.5) > 1e-4
    assert np.array_equal(labels[safe], m.predict(Xt)[safe])
    assert np.array_equal(labels, np.argmax(proba, axis=1))
    # the oracle on a sample
    desc = fi._desc
    idx = np.random.default_rng(0).choice(Xt.shape[0], 50_000, replace=False)
    np.testing.assert_allclose(proba[idx], oracle.predict(desc, Xt[idx], INFER_DEFAULT, "single"),
                               rtol=1e-5, atol=1e-6)
    assert np.array_equal(ids[idx].astype(np.uint32),
                          oracle.predict(desc, Xt[idx], INFER_LEAF_ID, "single"))


def test_c3_sklearn_regressor_exact_recipe_fp64():
    """RandomForestRegressor(200 trees, max_depth 20, min_samples_leaf 1) fit on 100,000
    make_regression rows (64 fp64 features, noise 0.1): 2.2e7 nodes in sparse storage.  Leaf ids
    bit-exact against scikit-learn's `apply` on 200,000 fp32-representable rows (scikit-learn
    casts inputs to fp32), and against the oracle on rows that only fp64 can hold."""
    from sklearn.datasets import make_regression
    from sklearn.ensemble import RandomForestRegressor

    X, y = make_regression(n_samples=100_000, n_features=64, noise=0.1, random_state=0)
    m = RandomForestRegressor(n_estimators=200, max_depth=20, min_samples_leaf=1, random_state=0,
                              n_jobs=-1).fit(X, y)
    fi = ForestInference.load_from_sklearn(m, precision="double")
    d = fi.describe()
    assert not fi.is_classifier and d["storage"] == 2 and d["n_trees"] == 200
    assert d["n_nodes_in"] > 15_000_000 and d["precision"] == 1
    desc = fi._desc
    torch = _torch()
    n = 200_000
    X32 = make_regression(n_samples=n, n_features=64, noise=0.1,
                          random_state=1)[0].astype(np.float32)
    Xd = torch.as_tensor(X32.astype(np.float64), device="cuda:0")
    ids = fi.apply(Xd).cpu().numpy()
    assert ids.shape == (n, 200)
    assert np.array_equal(ids.astype(np.int64), m.apply(X32))
    pred = fi.predict(Xd).cpu().numpy()
    assert pred.shape == (n, 1)
    np.testing.assert_allclose(pred[:, 0], m.predict(X32), rtol=1e-11, atol=1e-9)
    # rows with all 53 mantissa bits in use: only an fp64 comparison routes them right
    rng = np.random.default_rng(2)
    X64 = rng.standard_normal((20_000, 64))
    # ... some of them one ulp on either side of a threshold of the feature they sit in
    internal = np.nonzero(desc.node_kind != 0)[0]
    pick = rng.choice(internal, size=4000, replace=False)
    rows = rng.integers(0, X64.shape[0], size=pick.size)
    thr = desc.threshold[pick]
    X64[rows, desc.feature[pick]] = np.where(rng.random(pick.size) < 0.5, thr,
                                             np.nextafter(thr, np.inf))
    Xd64 = torch.as_tensor(X64, device="cuda:0")
    want_ids = oracle.predict(desc, X64, INFER_LEAF_ID, "double")
    want = oracle.predict(desc, X64, INFER_DEFAULT, "double")
    for layout in ("depth_first", "breadth_first"):
        fl = fi if layout == "depth_first" else ForestInference.load_from_treelite_model(
            desc, precision="double", layout=layout)
        assert np.array_equal(fl.apply(Xd64).cpu().numpy().astype(np.uint32), want_ids)
        got = fl.predict(Xd64).cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-12 * np.abs(want).max())
        del fl


def _c4_rows(n, seed):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, 128)).astype(np.float32)
    X[:, :8] = rng.integers(0, 32, size=(n, 8)).astype(np.float32)
    X[rng.random((n, 128)) < 0.05] = np.nan
    return X


def test_c4_categorical_multiclass_full_forest():
    """500 rounds x 10 classes = 5000 depth-6 trees, 128 fp32 features of which 8 categorical
    (32 categories, bitset tests), 5 % NaN routed by per-node default direction, softmax."""
    desc = synthetic_complete_forest(5000, 6, 128, seed=4, n_classes=10, n_categorical=8,
                                     n_categories=32)
    fi = ForestInference.load_from_treelite_model(desc)
    d = fi.describe()
    assert d["storage"] == 1 and d["row_quantization"] == 1 and d["n_trees"] == 5000
    torch = _torch()
    n = 200_000
    X = _c4_rows(n, 5)
    Xd = torch.as_tensor(X, device="cuda:0")
    proba = fi.predict_proba(Xd).cpu().numpy()
    assert proba.shape == (n, 10)
    np.testing.assert_allclose(proba.sum(axis=1), 1.0, rtol=1e-5)
    idx = np.random.default_rng(1).choice(n, 20_000, replace=False)
    idx[:3] = (0, n - 1, n // 2)
    want = oracle.predict(desc, X[idx], INFER_DEFAULT, "single")
    np.testing.assert_allclose(proba[idx], want, rtol=1e-5, atol=1e-6)
    labels = fi.predict(Xd).cpu().numpy()
    top2 = np.sort(want, axis=1)[:, -2:]
    safe = (top2[:, 1] - top2[:, 0]) > 1e-4
    assert np.array_equal(labels[idx][safe], np.argmax(want, axis=1)[safe])
    sub = idx[:2000]
    ids = fi.apply(Xd[torch.as_tensor(sub, device="cuda:0")]).cpu().numpy()
    assert np.array_equal(ids.astype(np.uint32),
                          oracle.predict(desc, X[sub], INFER_LEAF_ID, "single"))


def test_c5_depth10_512_features_full_forest():
    """2000 complete depth-10 trees over 512 fp32 features (the multi-GPU scale-out forest)."""
    desc = synthetic_complete_forest(2000, 10, 512, seed=6)
    fi = ForestInference.load_from_treelite_model(desc)
    d = fi.describe()
    assert d["storage"] == 1 and d["row_quantization"] == 1 and d["n_trees"] == 2000
    torch = _torch()
    n = 200_000
    g = torch.Generator(device="cuda:0")
    g.manual_seed(7)
    Xd = torch.randn((n, 512), generator=g, device="cuda:0", dtype=torch.float32)
    proba = fi.predict_proba(Xd)
    idx = torch.randint(0, n, (20_000,), generator=g, device="cuda:0")
    idx[:3] = torch.tensor([0, n - 1, n // 2], device="cuda:0")
    Xs = Xd[idx].cpu().numpy()
    np.testing.assert_allclose(proba[idx].cpu().numpy(),
                               oracle.predict(desc, Xs, INFER_PROBA2, "single"),
                               rtol=1e-5, atol=1e-6)
    ids = fi.apply(Xd[idx[:2000]]).cpu().numpy()
    assert np.array_equal(ids.astype(np.uint32),
                          oracle.predict(desc, Xs[:2000], INFER_LEAF_ID, "single"))
    # leaf ids -> leaf values -> sum -> sigmoid reproduces the scores on a slice
    m = 20_000
    all_ids = fi.apply(Xd[:m]).long()
    leaf = torch.as_tensor(desc.leaf_value.reshape(2000, -1), device="cuda:0")
    score = torch.sigmoid(leaf.gather(1, all_ids.t()).sum(dim=0))
    np.testing.assert_allclose(proba[:m, 1].cpu().numpy(), score.cpu().numpy(),
                               rtol=1e-5, atol=1e-6)
