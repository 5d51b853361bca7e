"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the golden fixtures.

Bars: leaf ids and class labels bit-exact; scores within rtol 1e-5 (fp32) / 1e-12 (fp64) with a
small absolute floor for values near zero (the reference's own boundary test uses rtol=1e-5,
atol=1e-6: python/cuml/tests/test_isolation_forest.py:751-762).
"""
import numpy as np
import pytest

from cuml_b200.fil import ForestInference, synthetic_complete_forest
from cuml_b200.fil._desc import (INFER_CLASS, INFER_DEFAULT, INFER_LEAF_ID, INFER_PER_TREE,
                                 INFER_PROBA2, OP_LE, OP_LT)
from oracle import oracle
from tests.helpers import load_golden, random_forest_desc, random_rows

pytestmark = pytest.mark.gpu

TOL = {"single": dict(rtol=1e-5, atol=1e-6), "double": dict(rtol=1e-12, atol=1e-13)}
CONFIGS = [("depth_first", "sparse"), ("breadth_first", "sparse"), ("layered", "sparse"),
           ("depth_first", "dense"), ("depth_first", "auto")]


def _torch():
    import torch

    return torch


def _dev(X, precision):
    torch = _torch()
    dt = torch.float32 if precision == "single" else torch.float64
    return torch.as_tensor(np.ascontiguousarray(X), device="cuda:0").to(dt)


def _tol(desc, precision):
    """Score tolerance: the relative bar of the parity contract plus an absolute floor that
    scales with the largest partial sum the forest can produce (results near zero come from
    cancellation of sums of that size, accumulated in another order than the oracle's)."""
    w = max(1, desc.leaf_vector_len)
    per_tree = [np.abs(desc.leaf_value[int(b) * w:int(e) * w]).max()
                for b, e in zip(desc.tree_offsets[:-1], desc.tree_offsets[1:])]
    scale = float(np.sum(per_tree))
    if desc.average_tree_output:
        scale /= max(1, desc.n_trees // max(1, desc.n_outputs if w == 1 else 1))
    base = TOL[precision]
    return dict(rtol=base["rtol"], atol=base["atol"] * max(1.0, scale))


def _all_kinds(desc, X, precision, layout, storage, chunk_size=None, host=False,
               quantize_rows=True, compact_nodes=True):
    """Run every output kind on the GPU and compare with the oracle."""
    tol = _tol(desc, precision)
    fi = ForestInference.load_from_treelite_model(desc, precision=precision, layout=layout,
                                                  storage=storage, quantize_rows=quantize_rows,
                                                  compact_nodes=compact_nodes)
    Xo = np.ascontiguousarray(X, np.float32 if precision == "single" else np.float64)
    Xd = Xo if host else _dev(Xo, precision)

    def get(a):
        return a if isinstance(a, np.ndarray) else a.cpu().numpy()

    ids = get(fi.apply(Xd, chunk_size=chunk_size))
    assert np.array_equal(ids.astype(np.uint32), oracle.predict(desc, Xo, INFER_LEAF_ID, precision))
    pt = get(fi.predict_per_tree(Xd, chunk_size=chunk_size))
    assert np.array_equal(pt, oracle.predict(desc, Xo, INFER_PER_TREE, precision))
    raw = get(fi._run(Xd, INFER_DEFAULT, chunk_size))
    want = oracle.predict(desc, Xo, INFER_DEFAULT, precision)
    np.testing.assert_allclose(raw, want, **tol)
    cls = get(fi._run(Xd, INFER_CLASS, chunk_size, threshold=0.5))
    want_cls = oracle.predict(desc, Xo, INFER_CLASS, precision, threshold=0.5)
    if desc.n_outputs == 1:
        safe = np.abs(want[:, 0] - 0.5) > 1e-4  # scores at the threshold may fall either way
    else:
        top2 = np.sort(want, axis=1)[:, -2:]
        safe = (top2[:, 1] - top2[:, 0]) > 1e-4 * np.maximum(1.0, np.abs(top2[:, 1]))
    assert np.array_equal(cls[safe], want_cls[safe])
    if desc.n_outputs == 1:
        p2 = get(fi._run(Xd, INFER_PROBA2, chunk_size))
        np.testing.assert_allclose(p2, oracle.predict(desc, Xo, INFER_PROBA2, precision), **tol)
    return fi


@pytest.mark.parametrize("layout,storage", CONFIGS)
@pytest.mark.parametrize("precision", ["single", "double"])
def test_random_forests_operators_nan(layout, storage, precision):
    desc = random_forest_desc(1, n_trees=23, max_depth=6, mixed_ops=True, integer_thresholds=True,
                              postproc="sigmoid")
    X = random_rows(2, 777, desc.n_features, np.float64, nan_frac=0.15, integer=True)
    _all_kinds(desc, X, precision, layout, storage)
    if storage == "sparse":  # the plain sparse kernel, which forests without a compact image use
        fi = _all_kinds(desc, X, precision, layout, storage, compact_nodes=False)
        assert fi.describe()["compact_image"] == 0


@pytest.mark.parametrize("precision", ["single", "double"])
def test_forests_over_a_thousand_features_and_more(precision):
    """A row tile of reals no longer fits shared memory, a tile of 16-bit ranks does: such forests
    keep dense storage and run the traversal over rank-quantised rows at every batch size (one
    row included) when a row visits enough nodes per feature to pay for ranking it; small
    forests stay sparse unless dense storage is asked for.  Without rank tables
    (quantize_rows=False) there is no dense kernel for them: sparse storage, and dense storage on
    request is refused."""
    from cuml_b200.fil import _lib

    for n_features, n_trees, n_rows in ((1100, 400, 1500), (2500, 620, 700)):
        desc = random_forest_desc(80 + n_features, n_trees=n_trees, n_features=n_features,
                                  max_depth=6, mixed_ops=True, postproc="sigmoid", p_leaf=0.05)
        X = random_rows(81, n_rows, n_features, np.float64, nan_frac=0.02)
        fi = _all_kinds(desc, X, precision, "depth_first", "auto")
        d = fi.describe()
        assert d["storage"] == 1 and d["row_quantization"] == 1, d
        assert "dense_q" in _lib.last_variant(), _lib.last_variant()
        _all_kinds(desc, X[:1], precision, "depth_first", "auto")
        sp = _all_kinds(desc, X[:300], precision, "depth_first", "auto", quantize_rows=False)
        assert sp.describe()["storage"] == 2
        with pytest.raises(Exception):
            ForestInference.load_from_treelite_model(desc, precision=precision, storage="dense",
                                                     quantize_rows=False)
        # few trees: ranking 1100 or 2500 features per row costs more than the walks save
        small = random_forest_desc(82, n_trees=12, n_features=n_features, max_depth=6)
        fi = _all_kinds(small, X[:300], precision, "depth_first", "auto")
        assert fi.describe()["storage"] == 2
        fi = _all_kinds(small, X[:33], precision, "depth_first", "dense")
        assert fi.describe()["storage"] == 1 and "dense_q" in _lib.last_variant()


@pytest.mark.parametrize("precision", ["single", "double"])
@pytest.mark.parametrize("quantize_rows", [True, False])
def test_dense_with_and_without_row_quantisation(precision, quantize_rows):
    # scalar leaves, multi-class scalar leaves and vector leaves through both dense kernels
    for seed, kw in ((1, dict(postproc="sigmoid")), (2, dict(n_outputs=3, postproc="softmax")),
                     (3, dict(n_outputs=4, vector=True, average=True))):
        desc = random_forest_desc(seed, n_trees=21, max_depth=6, mixed_ops=True, **kw)
        X = random_rows(seed, 900, desc.n_features, np.float64, nan_frac=0.1)
        fi = _all_kinds(desc, X, precision, "depth_first", "dense", quantize_rows=quantize_rows)
        assert fi.describe()["row_quantization"] == int(quantize_rows)
        # batches this small split the forest over CTAs of the plain kernel; an explicit chunk
        # size asks for the regular path (rank pre-pass + quantised walk when it exists)
        _all_kinds(desc, X, precision, "depth_first", "dense", quantize_rows=quantize_rows,
                   chunk_size=4)


@pytest.mark.parametrize("precision", ["single", "double"])
def test_sparse_compact_image_deep_ragged_trees(precision):
    """The kernel over the compact image on what it is for: ragged trees much deeper than the
    heap of top levels, rows made of the thresholds and their neighbours (fp64: the float bound
    in the 8-byte node cannot decide them, the exact threshold must), NaN and infinities,
    single-leaf trees in the same forest, batches that fill 32-, 64- and 128-row tiles with a
    ragged tail, and a tree count that leaves the last batch of heaps half empty."""
    from cuml_b200.fil import _lib, concatenate

    deep = random_forest_desc(35, n_trees=37, n_features=9, max_depth=16, p_leaf=0.25,
                              mixed_ops=True, postproc="sigmoid")
    stumps = random_forest_desc(36, n_trees=3, n_features=9, max_depth=0, postproc="sigmoid")
    desc = concatenate([deep, stumps])
    dt = np.float32 if precision == "single" else np.float64
    thr = desc.threshold[desc.node_kind == 1]
    rng = np.random.default_rng(4)
    vals = np.concatenate([thr, np.nextafter(thr, np.inf), np.nextafter(thr, -np.inf),
                           thr.astype(np.float32).astype(np.float64),
                           [np.nan, np.inf, -np.inf, 0.0, -0.0]]).astype(dt)
    for n in (70, 9_600, 23_001):
        X = rng.choice(vals, size=(n, 9)).astype(dt)
        X[: n // 2] = random_rows(5, n // 2, 9, dt, nan_frac=0.05)
        fi = _all_kinds(desc, X, precision, "depth_first", "sparse")
        d = fi.describe()
        assert d["compact_image"] == 1 and d["top_levels"] >= 4
        assert _lib.last_variant().startswith("sparse_compact_kernel<")
    # other heap depths (a tuning option) give the same answers
    X = rng.choice(vals, size=(5000, 9)).astype(dt)
    for levels in (1, 3, 9, 10):
        fi = _all_kinds(desc, X, precision, "depth_first", "sparse", compact_nodes=levels)
        assert fi.describe()["top_levels"] == levels
    # vector leaves and several classes through the same kernel
    vec = random_forest_desc(37, n_trees=21, n_outputs=3, vector=True, average=True, max_depth=13,
                             p_leaf=0.12)
    _all_kinds(vec, random_rows(6, 3000, vec.n_features, dt), precision, "breadth_first", "sparse")
    multi = random_forest_desc(38, n_trees=30, n_outputs=4, max_depth=12, p_leaf=0.12,
                               postproc="softmax")
    _all_kinds(multi, random_rows(7, 3000, multi.n_features, dt), precision, "layered", "sparse")


def test_row_quantisation_edge_values():
    # rows made of the thresholds themselves, their neighbours, infinities, signed zeros,
    # denormals and NaN: ranks must reproduce every comparison exactly
    for prec, dt in (("single", np.float32), ("double", np.float64)):
        desc = random_forest_desc(21, n_trees=30, n_features=4, max_depth=6, mixed_ops=True)
        thr = desc.threshold[desc.node_kind == 1].astype(dt)
        vals = np.concatenate([thr, np.nextafter(thr, dt(np.inf)), np.nextafter(thr, dt(-np.inf)),
                               np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45,
                                         np.finfo(dt).max, np.finfo(dt).min, np.finfo(dt).tiny],
                                        dt)])
        X = np.random.default_rng(5).choice(vals, size=(5000, 4)).astype(dt)
        _all_kinds(desc, X, prec, "depth_first", "dense", chunk_size=8)  # quantised walk
        _all_kinds(desc, X, prec, "depth_first", "dense")               # small-batch split path


def test_row_quantisation_nan_free_and_nan_tiles():
    # a batch whose first tiles hold no NaN and whose last tiles do: both code paths in one launch
    desc = random_forest_desc(23, n_trees=40, n_features=9, max_depth=7)
    X = random_rows(6, 4000, desc.n_features, np.float32, nan_frac=0.0)
    X[3000:] = random_rows(7, 1000, desc.n_features, np.float32, nan_frac=0.3)
    for chunk_size in (1, 2, 8):  # 32-, 64- and 256-row tiles of the quantised walk
        _all_kinds(desc, X, "single", "depth_first", "dense", chunk_size=chunk_size)
    _all_kinds(desc, X, "single", "depth_first", "dense")


@pytest.mark.parametrize("layout,storage", CONFIGS)
@pytest.mark.parametrize("big", [False, True])
def test_categorical(layout, storage, big):
    desc = random_forest_desc(3 + big, n_trees=17, max_depth=5, categorical=True,
                              big_categories=big, mixed_ops=True, n_outputs=3, postproc="softmax")
    X = random_rows(4, 500, desc.n_features, np.float32, nan_frac=0.1, categories=75 if big else 22)
    _all_kinds(desc, X, "single", layout, storage)
    _all_kinds(desc, X, "double", layout, storage)
    if storage == "sparse":
        _all_kinds(desc, X, "single", layout, storage, compact_nodes=False)
        _all_kinds(desc, X, "double", layout, storage, compact_nodes=False)


@pytest.mark.parametrize("layout,storage", CONFIGS)
@pytest.mark.parametrize("precision", ["single", "double"])
def test_vector_leaves(layout, storage, precision):
    # five and eleven outputs: more than the sums a thread keeps in registers, added to shared
    # memory four at a time with a remainder of one and of three
    for n_outputs in (5, 8, 11):  # (eight: vectors that load 16 bytes at a time)
        desc = random_forest_desc(5, n_trees=13, n_outputs=n_outputs, vector=True, average=True)
        X = random_rows(6, 300, desc.n_features, np.float32)
        _all_kinds(desc, X, precision, layout, storage)
        if storage == "sparse":
            _all_kinds(desc, X, precision, layout, storage, compact_nodes=False)


@pytest.mark.parametrize("post", ["identity", "sigmoid", "exponential", "logarithm_one_plus_exp",
                                  "signed_square", "hinge", "exponential_standard_ratio"])
def test_postprocessors_one_output(post):
    desc = random_forest_desc(40, n_trees=6, postproc=post, base=True, average=True)
    X = random_rows(5, 200, desc.n_features, np.float32, nan_frac=0.0)
    for storage in ("dense", "sparse"):
        fi = ForestInference.load_from_treelite_model(desc, storage=storage)
        got = fi._run(_dev(X, "single"), INFER_DEFAULT, None).cpu().numpy()
        want = oracle.predict(desc, X, INFER_DEFAULT, "single")
        if post == "hinge":
            safe = np.abs(oracle.predict(
                random_forest_desc(40, n_trees=6, postproc="identity", base=True, average=True),
                X, INFER_DEFAULT, "single")) > 1e-5
            assert np.array_equal(got[safe], want[safe])
        else:
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("post", ["softmax", "multiclass_ova"])
def test_postprocessors_multiclass(post):
    desc = random_forest_desc(41, n_trees=12, n_outputs=4, postproc=post, base=True)
    X = random_rows(5, 200, desc.n_features, np.float32, nan_frac=0.0)
    for storage in ("dense", "sparse"):
        _all_kinds(desc, X, "single", "depth_first", storage)


@pytest.mark.parametrize("n_rows", [0, 1, 31, 32, 33, 127, 129, 1000, 2368, 2369, 2400, 5000])
def test_ragged_batch_sizes(n_rows):
    desc = random_forest_desc(50, n_trees=9, max_depth=5, n_outputs=2, postproc="softmax")
    X = random_rows(7, max(n_rows, 1), desc.n_features, np.float32)[:n_rows]
    for storage in ("dense", "sparse"):
        fi = ForestInference.load_from_treelite_model(desc, storage=storage)
        got = fi.predict_proba(_dev(X, "single").reshape(n_rows, desc.n_features)).cpu().numpy()
        assert got.shape == (n_rows, 2)
        if n_rows:
            np.testing.assert_allclose(got, oracle.predict(desc, X, INFER_DEFAULT, "single"),
                                       rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("chunk_size", [1, 2, 4, 8, 16, 32])
def test_chunk_sizes_give_identical_ids(chunk_size):
    desc = random_forest_desc(51, n_trees=19, max_depth=6)
    X = random_rows(8, 3000, desc.n_features, np.float32)
    for storage in ("dense", "sparse"):
        _all_kinds(desc, X, "single", "depth_first", storage, chunk_size=chunk_size)


def test_single_leaf_trees_and_tiny_forests():
    for depth in (0, 1):
        desc = random_forest_desc(52, n_trees=3, max_depth=depth, p_leaf=0.0)
        X = random_rows(9, 70, desc.n_features, np.float32)
        for storage in ("dense", "sparse"):
            _all_kinds(desc, X, "single", "depth_first", storage)
            _all_kinds(desc, X, "double", "depth_first", storage)
    # larger batches of the same tiny forests take the quantised path when it exists
    desc = random_forest_desc(52, n_trees=3, max_depth=1, p_leaf=0.0)
    X = random_rows(9, 12000, desc.n_features, np.float32)
    for precision in ("single", "double"):
        _all_kinds(desc, X, precision, "depth_first", "dense")


def test_row_stride_and_host_buffers():
    torch = _torch()
    desc = random_forest_desc(53, n_trees=11, max_depth=5, n_features=6)
    wide = torch.as_tensor(random_rows(10, 500, 10, np.float32), device="cuda:0")
    view = wide[:, :6]  # rows 10 elements apart, 6 used
    assert view.stride(0) == 10
    fi = ForestInference.load_from_treelite_model(desc)
    got = fi.apply(view).cpu().numpy()
    X = view.cpu().numpy()
    assert np.array_equal(got.astype(np.uint32), oracle.predict(desc, X, INFER_LEAF_ID, "single"))
    # host buffers take the copy-predict-copy pipeline inside the library
    _all_kinds(desc, X, "single", "depth_first", "auto", host=True)
    _all_kinds(desc, X, "double", "depth_first", "sparse", host=True)


def test_pageable_host_arrays_take_the_staged_pipeline(lib):
    """An ordinary NumPy array of several hundred MB: the library gathers row blocks into its own
    pinned staging buffers with a few host threads (three slots, 64 MiB blocks, so slots are
    reused) instead of leaving the staging to the driver.  Leaf ids must equal the device path bit
    for bit and scores within the parity tolerance (row blocks choose their own tile shapes, and
    with them the order of the sums); a strided input through the C ABI as well."""
    import ctypes as C

    torch = _torch()
    desc = synthetic_complete_forest(60, 6, 256, seed=12)
    fi = ForestInference.load_from_treelite_model(desc)
    rng = np.random.default_rng(13)
    n = 330_000  # 338 MB of fp32 rows: six blocks
    X = rng.standard_normal((n, 256), dtype=np.float32)
    X[::1000, 7] = np.nan
    want = fi.predict_proba(torch.as_tensor(X, device="cuda:0")).cpu().numpy()
    got = fi.predict_proba(X)
    assert isinstance(got, np.ndarray)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-7)
    idx = rng.choice(n, 3000, replace=False)
    np.testing.assert_allclose(got[idx], oracle.predict(desc, X[idx], INFER_PROBA2, "single"),
                               rtol=1e-5, atol=1e-6)
    ids = fi.apply(X[:70_000])  # 72 MB: two blocks, uint32 outputs of 240 bytes per row
    assert np.array_equal(ids, fi.apply(torch.as_tensor(X[:70_000], device="cuda:0")).cpu().numpy())
    # rows 256 elements apart of which the forest uses the first 200
    narrow = synthetic_complete_forest(40, 5, 200, seed=14)
    fn = ForestInference.load_from_treelite_model(narrow)
    out = np.empty((n, 2), np.float32)
    rc = lib.b2fil_predict_host(fn.forest.handle, INFER_PROBA2, X.ctypes.data, n, 256,
                                out.ctypes.data, 0, 0.5)
    assert rc == 0, lib.b2fil_last_error()
    ref = fn.predict_proba(torch.as_tensor(np.ascontiguousarray(X[:, :200]), device="cuda:0"))
    np.testing.assert_allclose(out, ref.cpu().numpy(), rtol=1e-6, atol=1e-7)
    # pinned arrays keep the direct path and agree too
    Xp = torch.empty((100_000, 256), dtype=torch.float32, pin_memory=True)
    Xp.copy_(torch.as_tensor(X[:100_000]))
    np.testing.assert_allclose(fi.predict_proba(Xp.numpy()), want[:100_000], rtol=1e-6, atol=1e-7)


def test_golden_rfc_depth8():
    desc, X, exp = load_golden("rfc_depth8")
    for storage in ("dense", "sparse"):
        fi = ForestInference.load_from_treelite_model(desc, storage=storage)
        assert type(fi).__name__ == "ForestInferenceClassifier"
        Xd = _dev(X, "single")
        assert np.array_equal(fi.apply(Xd).cpu().numpy().astype(np.int64), exp["leaf_ids"])
        np.testing.assert_allclose(fi.predict_proba(Xd).cpu().numpy(), exp["proba"],
                                   rtol=1e-5, atol=1e-6)
        pred = fi.predict(Xd).cpu().numpy()
        safe = np.abs(exp["proba"][:, 0] - 0.5) > 1e-4
        assert np.array_equal(pred[safe].astype(np.int64), exp["labels"][safe])
        # predict == argmax(predict_proba): python/cuml/tests/test_random_forest.py:853-855
        assert np.array_equal(pred, np.argmax(fi.predict_proba(Xd).cpu().numpy(), axis=1))


def test_golden_rfr_depth20_fp64():
    desc, X, exp = load_golden("rfr_depth20")
    for layout in ("depth_first", "breadth_first", "layered"):
        fi = ForestInference.load_from_treelite_model(desc, precision="double", layout=layout)
        assert type(fi).__name__ == "ForestInferenceRegressor"
        assert fi.describe()["storage"] == 2
        Xd = _dev(X, "double")
        assert np.array_equal(fi.apply(Xd).cpu().numpy().astype(np.int64), exp["leaf_ids"])
        got = fi.predict(Xd).cpu().numpy()
        assert got.shape == (X.shape[0], 1)
        np.testing.assert_allclose(got[:, 0], exp["values"], rtol=1e-12, atol=1e-12)


def test_golden_gbc_3class_and_missing():
    desc, X, exp = load_golden("gbc_3class")
    fi = ForestInference.load_from_treelite_model(desc, precision="double")
    np.testing.assert_allclose(fi.predict_proba(_dev(X, "double")).cpu().numpy(), exp["proba"],
                               rtol=1e-12, atol=1e-13)
    desc, X, exp = load_golden("rfc_missing")
    for storage in ("dense", "sparse"):
        fi = ForestInference.load_from_treelite_model(desc, storage=storage)
        Xd = _dev(X, "single")
        assert np.array_equal(fi.apply(Xd).cpu().numpy().astype(np.int64), exp["leaf_ids"])
        np.testing.assert_allclose(fi.predict_proba(Xd).cpu().numpy(), exp["proba"],
                                   rtol=1e-5, atol=1e-6)


def test_sklearn_models_trained_here():
    from sklearn.datasets import make_classification
    from sklearn.ensemble import GradientBoostingClassifier, RandomForestClassifier

    X, y = make_classification(n_samples=3000, n_features=32, n_informative=16, n_classes=2,
                               random_state=0)
    X = X.astype(np.float32)
    m = RandomForestClassifier(n_estimators=100, max_depth=8, random_state=0, n_jobs=-1).fit(X, y)
    Xt = make_classification(n_samples=20000, n_features=32, n_informative=16, n_classes=2,
                             random_state=1)[0].astype(np.float32)
    fi = ForestInference.load_from_sklearn(m)
    assert fi.is_classifier and fi.describe()["storage"] == 1
    assert np.array_equal(fi.apply(Xt).astype(np.int64), m.apply(Xt))
    np.testing.assert_allclose(fi.predict_proba(Xt), m.predict_proba(Xt), rtol=1e-5, atol=1e-6)
    g = GradientBoostingClassifier(n_estimators=30, max_depth=3, random_state=0).fit(X[:, :8], y)
    fg = ForestInference.load_from_sklearn(g, precision="double")
    Xg = Xt[:, :8].astype(np.float64)
    np.testing.assert_allclose(fg.predict_proba(Xg), g.predict_proba(Xg), rtol=1e-12, atol=1e-13)


def _config_forest(name):
    if name == "c2":  # 1000 complete depth-8 trees, 256 features, sigmoid (smaller row count)
        return synthetic_complete_forest(1000, 8, 256, seed=2), 256, None, 0.0
    if name == "c4":  # 10-class boosted forest, depth 6, 8 categorical features, 5 % NaN
        return (synthetic_complete_forest(500, 6, 128, seed=4, n_classes=10, n_categorical=8,
                                          n_categories=32), 128, 32, 0.05)
    if name == "c5":  # complete depth-10 trees, 512 features
        return synthetic_complete_forest(64, 10, 512, seed=6), 512, None, 0.0
    raise KeyError(name)


@pytest.mark.parametrize("name", ["c2", "c4", "c5"])
def test_benchmark_config_shapes(name):
    desc, F, cats, nan_frac = _config_forest(name)
    rng = np.random.default_rng(3)
    n = 12000  # enough row tiles for the regular (quantised) path
    X = rng.standard_normal((n, F)).astype(np.float32)
    if cats:
        X[:, :8] = rng.integers(0, cats, size=(n, 8)).astype(np.float32)
        X[rng.random((n, F)) < nan_frac] = np.nan
    fi = ForestInference.load_from_treelite_model(desc)
    assert fi.describe()["storage"] == 1
    Xd = _dev(X, "single")
    proba = fi.predict_proba(Xd).cpu().numpy()
    kind = INFER_PROBA2 if desc.n_outputs == 1 else INFER_DEFAULT
    np.testing.assert_allclose(proba, oracle.predict(desc, X, kind, "single"), rtol=1e-5, atol=1e-6)
    ids = fi.apply(Xd[:1500]).cpu().numpy()
    assert np.array_equal(ids.astype(np.uint32),
                          oracle.predict(desc, X[:1500], INFER_LEAF_ID, "single"))
    # the same forest with `<=` tests and sparse storage agrees as well
    if name == "c2":
        desc_le = synthetic_complete_forest(1000, 8, 256, seed=2, op=OP_LE)
        fl = ForestInference.load_from_treelite_model(desc_le, storage="sparse",
                                                      layout="breadth_first")
        ids = fl.apply(Xd[:1500]).cpu().numpy()
        assert np.array_equal(ids.astype(np.uint32),
                              oracle.predict(desc_le, X[:1500], INFER_LEAF_ID, "single"))


def test_full_size_c2_properties():
    """The headline workload at full size (10 M rows x 256 features, 1000 depth-8 trees):
    a random sample of rows against the oracle, and a sum-of-leaves check that ties the leaf-id
    output to the score output on a slice."""
    torch = _torch()
    desc = synthetic_complete_forest(1000, 8, 256, seed=2)
    fi = ForestInference.load_from_treelite_model(desc)
    n = 10_000_000
    g = torch.Generator(device="cuda:0")
    g.manual_seed(3)
    X = torch.randn((n, 256), generator=g, device="cuda:0", dtype=torch.float32)
    proba = fi.predict_proba(X)
    assert proba.shape == (n, 2)
    idx = torch.randint(0, n, (4096,), generator=g, device="cuda:0")
    idx[:3] = torch.tensor([0, n - 1, n // 2], device="cuda:0")
    Xs = X[idx].cpu().numpy()
    np.testing.assert_allclose(proba[idx].cpu().numpy(),
                               oracle.predict(desc, Xs, INFER_PROBA2, "single"),
                               rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(proba.sum(dim=1).cpu().numpy(), 1.0, rtol=1e-6)
    # leaf ids -> leaf values -> sum -> sigmoid reproduces the scores
    m = 200_000
    ids = fi.apply(X[:m]).long()  # heap ids of the complete trees
    leaf = torch.as_tensor(desc.leaf_value.reshape(1000, -1), device="cuda:0")
    vals = leaf.gather(1, ids.t()).t()  # (m, 1000) float64
    score = torch.sigmoid(vals.sum(dim=1))
    np.testing.assert_allclose(proba[:m, 1].cpu().numpy(), score.cpu().numpy(), rtol=1e-5, atol=1e-6)
    per_tree = fi.predict_per_tree(X[:m])
    assert torch.equal(per_tree.double(), vals)


def test_status_word_and_launch_counter(lib):
    import ctypes as C

    desc = random_forest_desc(60, n_trees=5)
    fi = ForestInference.load_from_treelite_model(desc, storage="dense", quantize_rows=False)
    before = lib.b2fil_kernel_launches()
    fi.apply(_dev(random_rows(1, 100, desc.n_features), "single"))
    _torch().cuda.synchronize()
    assert lib.b2fil_kernel_launches() == before + 1
    # with rank quantisation a prediction is a pre-pass plus a traversal kernel per row chunk
    fq = ForestInference.load_from_treelite_model(desc, storage="dense")
    before = lib.b2fil_kernel_launches()
    fq.apply(_dev(random_rows(1, 20000, desc.n_features), "single"))
    _torch().cuda.synchronize()
    assert lib.b2fil_kernel_launches() == before + 2
    # a small batch splits the forest over CTAs: walk + finish kernel for reduced outputs
    before = lib.b2fil_kernel_launches()
    fq.predict_proba(_dev(random_rows(1, 100, desc.n_features), "single")) if fq.is_classifier \
        else fq.predict(_dev(random_rows(1, 100, desc.n_features), "single"))
    _torch().cuda.synchronize()
    assert lib.b2fil_kernel_launches() in (before + 1, before + 2)
    st = C.c_int32(-1)
    assert lib.b2fil_forest_status(fi.forest.handle, C.byref(st)) == 0 and st.value == 0


def test_pickle_round_trip():
    import pickle

    desc = random_forest_desc(61, n_trees=7, n_outputs=3, vector=True, average=True)
    fi = ForestInference.load_from_treelite_model(desc)
    X = _dev(random_rows(2, 200, desc.n_features), "single")
    a = fi.predict_proba(X).cpu().numpy()
    fi2 = pickle.loads(pickle.dumps(fi))
    assert np.array_equal(a, fi2.predict_proba(X).cpu().numpy())


def test_sharded_prediction_over_available_gpus(lib):
    """Model replicated, rows sharded, results gathered on the first device by peer copies: on
    every device the box has (one process drives them all)."""
    import ctypes as C

    torch = _torch()
    from cuml_b200.fil.multi_gpu import ShardedForestInference

    n_dev = min(torch.cuda.device_count(), 8)
    desc = random_forest_desc(80, n_trees=31, n_features=10, max_depth=6, n_outputs=3,
                              postproc="softmax")
    fi = ForestInference.load_from_treelite_model(desc, device_id=0)
    sh = ShardedForestInference(fi, list(range(n_dev)))
    X = random_rows(9, 5003, 10, np.float32, nan_frac=0.05)
    shards = sh.scatter(X)
    assert sum(s.shape[0] for s in shards) == 5003
    proba = sh.predict_proba(shards).cpu().numpy()
    np.testing.assert_allclose(proba, oracle.predict(desc, X, INFER_DEFAULT, "single"),
                               rtol=1e-5, atol=1e-6)
    ids = sh.apply(shards).cpu().numpy()
    assert np.array_equal(ids.astype(np.uint32), oracle.predict(desc, X, INFER_LEAF_ID, "single"))
    cls = sh.predict(shards).cpu().numpy()
    assert np.array_equal(cls, np.argmax(proba, axis=1))
    t = sh.last_timing()
    assert t["wall_ms"] > 0 and t["compute_ms"] > 0 and t["gather_direct"] in (0, 1)
    for f in sh._forests[1:]:
        assert f.info.clone_src_device == 0 and f.info.peer_direct in (0, 1)
    assert fi.forest.info.peer_direct == -1
    # empty shards and a quantised forest large enough for the regular path on every device
    big = synthetic_complete_forest(64, 6, 16, seed=3)
    fb = ForestInference.load_from_treelite_model(big, device_id=0)
    shb = ShardedForestInference(fb, list(range(n_dev)))
    Xb = np.random.default_rng(4).standard_normal((24_000 * n_dev + 17, 16)).astype(np.float32)
    got = shb.predict_proba(shb.scatter(Xb)).cpu().numpy()
    np.testing.assert_allclose(got, oracle.predict(big, Xb, INFER_PROBA2, "single"),
                               rtol=1e-5, atol=1e-6)
    parts = shb.scatter(Xb[:3])  # fewer rows than devices: some shards are empty
    got = shb.apply(parts).cpu().numpy()
    assert np.array_equal(got.astype(np.uint32), oracle.predict(big, Xb[:3], INFER_LEAF_ID, "single"))
    if n_dev > 1:
        assert lib.b2fil_enable_peer_access(0, 1) in (0, 1)
    assert lib.b2fil_enable_peer_access(0, 99) == -1


def test_sharded_prediction_from_two_threads_in_opposite_device_order():
    """Two host threads that hand the same forests to the sharded call in opposite orders must
    both finish (the forests' locks are taken in a fixed order)."""
    import threading

    torch = _torch()
    from cuml_b200.fil.multi_gpu import ShardedForestInference

    n_dev = min(torch.cuda.device_count(), 8)
    desc = random_forest_desc(81, n_trees=12, n_features=6, max_depth=5)
    fi = ForestInference.load_from_treelite_model(desc, device_id=0)
    sh = ShardedForestInference(fi, list(range(n_dev)))
    X = random_rows(3, 4000, 6, np.float32)
    want = oracle.predict(desc, X, INFER_LEAF_ID, "single")
    import ctypes as C

    lib = sh._lib
    order = list(range(n_dev))
    results, errors = {}, []

    def call(devs):
        """The C-ABI call with the forests listed in the order `devs`; the output lives on the
        first listed device and holds the shards in that order."""
        parts = {d: p for d, p in zip(order, sh.scatter(X))}
        for d in order:
            torch.cuda.synchronize(d)
        rows = [int(parts[d].shape[0]) for d in devs]
        out = torch.empty((sum(rows), desc.n_trees), dtype=torch.int32, device=f"cuda:{devs[0]}")
        handles = (C.c_void_p * n_dev)(*[sh._forests[d].handle for d in devs])
        xs = (C.c_void_p * n_dev)(*[parts[d].data_ptr() for d in devs])
        counts = (C.c_int64 * n_dev)(*rows)
        rc = lib.b2fil_predict_sharded(handles, n_dev, INFER_LEAF_ID, xs, counts, 6,
                                       out.data_ptr(), 0, 0.5)
        assert rc == 0, lib.b2fil_last_error()
        pieces = np.split(out.cpu().numpy(), np.cumsum(rows)[:-1])
        return np.concatenate([pieces[devs.index(d)] for d in order])

    def work(name, devs):
        try:
            for _ in range(20):
                results[name] = call(devs)
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    ts = [threading.Thread(target=work, args=("a", order)),
          threading.Thread(target=work, args=("b", order[::-1]))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in ts), "sharded calls blocked each other"
    assert not errors, errors
    for name in ("a", "b"):
        assert np.array_equal(results[name].astype(np.uint32), want)


def test_bounded_wait_runs_out_and_is_reported_once(lib):
    """A wait inside a kernel that nothing ends gives up after its limit, the kernel returns, the
    forest's status word says so, the host call reports B2FIL_ERR_TIMEOUT once, and the device
    keeps working.  (The wait is on an mbarrier that never receives its arrival; the limit is 16
    tries of a few microseconds, so nothing hangs.)"""
    import ctypes as C

    torch = _torch()
    desc = random_forest_desc(62, n_trees=5)
    fi = ForestInference.load_from_treelite_model(desc)
    X = _dev(random_rows(1, 300, desc.n_features), "single")
    before = fi.apply(X).cpu().numpy()
    st = C.c_int32(-1)
    assert lib.b2fil_forest_status(fi.forest.handle, C.byref(st)) == 0 and st.value == 0
    side = torch.cuda.Stream()  # a non-blocking stream: the status call must wait for it too
    assert lib.b2fil_forest_selftest_timeout(fi.forest.handle, 16, side.cuda_stream) == 0
    rc = lib.b2fil_forest_status(fi.forest.handle, C.byref(st))
    assert rc == -7 and st.value == 5
    assert b"ran out" in lib.b2fil_last_error()
    with pytest.raises(Exception) as ei:
        lib.b2fil_forest_selftest_timeout(fi.forest.handle, 16, None)
        fi.check_status()
    assert getattr(ei.value, "code", None) == -7
    # reported once: the word is clear again and predictions are unaffected
    assert lib.b2fil_forest_status(fi.forest.handle, C.byref(st)) == 0 and st.value == 0
    assert np.array_equal(fi.apply(X).cpu().numpy(), before)
    assert lib.b2fil_forest_selftest_timeout(fi.forest.handle, 0, None) == -1
    assert lib.b2fil_forest_selftest_timeout(None, 4, None) == -1


def test_last_variant_names_the_kernels(lib):
    from cuml_b200.fil import _lib

    desc = synthetic_complete_forest(100, 8, 64, seed=2)
    fi = ForestInference.load_from_treelite_model(desc)
    rng = np.random.default_rng(0)
    # 256-row tiles on every SM: the shape of large batches
    fi.predict_proba(_dev(rng.standard_normal((60_000, 64)).astype(np.float32), "single"))
    v = _lib.last_variant()
    assert v.startswith("quantise_kernel<float> + dense_q_top_kernel<float,scalar,NT=6,DEPTH=8>")
    # fewer rows than that: 128-row tiles and more tree groups
    fi.predict_proba(_dev(rng.standard_normal((30_000, 64)).astype(np.float32), "single"))
    v = _lib.last_variant()
    assert v.startswith("quantise_kernel<float> + dense_q_top_kernel<float,scalar,NT=6,DEPTH=8> R=128")
    fi.predict_proba(_dev(rng.standard_normal((64, 64)).astype(np.float32), "single"))
    v = _lib.last_variant()
    assert v.startswith("dense_kernel<float,scalar") and "forest_splits=" in v
    sp = ForestInference.load_from_treelite_model(desc, storage="sparse")
    sp.apply(_dev(rng.standard_normal((500, 64)).astype(np.float32), "single"))
    assert _lib.last_variant().startswith("sparse_compact_kernel<float,leaf_id,NT=4,TOP=8>")
    sp = ForestInference.load_from_treelite_model(desc, storage="sparse", compact_nodes=False)
    sp.apply(_dev(rng.standard_normal((500, 64)).astype(np.float32), "single"))
    assert _lib.last_variant().startswith("sparse_kernel<float,node8,leaf_id")


def test_quantised_categorical_edge_values():
    """Categorical features on the rank-quantised path: categories that are negative, fractional
    (truncated), beyond the 32-bit set, huge, infinite or NaN must route like the oracle says."""
    desc = synthetic_complete_forest(40, 5, 12, seed=9, n_classes=3, n_categorical=4,
                                     n_categories=32)
    rng = np.random.default_rng(10)
    n = 6000
    X = rng.standard_normal((n, 12)).astype(np.float32)
    cats = np.array([-1.0, -0.5, 0.0, 0.9, 1.0, 1.5, 30.99, 31.0, 31.5, 32.0, 33.0, 1e6, 4e4,
                     np.inf, -np.inf, np.nan, 16777216.0, 3e9], np.float32)
    X[:, :4] = rng.choice(cats, size=(n, 4))
    X[rng.random((n, 12)) < 0.03] = np.nan
    for precision in ("single", "double"):
        fi = _all_kinds(desc, X, precision, "depth_first", "dense", chunk_size=4)
        assert fi.describe()["row_quantization"] == 1
        _all_kinds(desc, X, precision, "depth_first", "dense")
        _all_kinds(desc, X, precision, "depth_first", "dense", quantize_rows=False)


def test_load_from_model_files(tmp_path):
    import json

    from cuml_b200.fil.loaders import save_desc
    from cuml_b200.fil.treelite_json import to_treelite_json

    desc = random_forest_desc(90, n_trees=12, n_features=7, max_depth=5, categorical=True,
                              n_outputs=3, postproc="softmax")
    X = random_rows(11, 400, 7, np.float32, categories=22)
    want = oracle.predict(desc, X, INFER_DEFAULT, "single")
    p1 = tmp_path / "forest.npz"
    save_desc(desc, str(p1))
    p2 = tmp_path / "treelite_dump.json"
    p2.write_text(json.dumps(to_treelite_json(desc)))
    for path, kind in ((p1, None), (p2, "treelite_json"), (p2, None)):
        fi = ForestInference.load(str(path), model_type=kind, is_classifier=True)
        np.testing.assert_allclose(fi.predict_proba(X), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("fmt", ["xgboost_json", "xgboost_ubjson", "lightgbm"])
@pytest.mark.parametrize("n_classes", [1, 4])
def test_model_files_of_other_libraries_on_the_gpu(tmp_path, fmt, n_classes):
    """Multi-tree, multi-class model files with categorical tests and missing values, written in
    the XGBoost JSON / UBJSON and LightGBM text formats (by this library's own writers: neither
    package is installed), loaded through ForestInference.load(path): scores and leaf ids of the
    GPU against the oracle on the same loaded description, in both storages."""
    import json

    from cuml_b200.fil import ubjson
    from cuml_b200.fil.lightgbm_txt import to_lightgbm_text
    from cuml_b200.fil.loaders import load_file
    from cuml_b200.fil.xgboost_json import to_xgboost_json
    from tests.helpers import lightgbm_style_desc, xgboost_style_desc

    if fmt == "lightgbm":
        src = lightgbm_style_desc(30 + n_classes, n_trees=40, n_features=11, max_depth=7,
                                  n_classes=n_classes)
        path = tmp_path / "model.txt"
        path.write_text(to_lightgbm_text(src, f"multiclass num_class:{n_classes}"
                                         if n_classes > 1 else "binary sigmoid:1.5"))
        precision = "double"
    else:
        src = xgboost_style_desc(20 + n_classes, n_trees=40, n_features=11, max_depth=7,
                                 n_classes=n_classes)
        obj = to_xgboost_json(src, "multi:softprob" if n_classes > 1 else "binary:logistic")
        if fmt == "xgboost_json":
            path = tmp_path / "model.json"
            path.write_text(json.dumps(obj))
        else:
            path = tmp_path / "model.ubj"
            path.write_bytes(ubjson.dumps(obj))
        precision = "single"
    loaded = load_file(str(path))
    dt = np.float32 if precision == "single" else np.float64
    X = random_rows(13, 3000, 11, dt, nan_frac=0.08, categories=22)
    kind = INFER_PROBA2 if n_classes == 1 else INFER_DEFAULT
    want = oracle.predict(loaded, X, kind, precision)
    # the file says what the source forest says
    np.testing.assert_allclose(want, oracle.predict(src, X, kind, precision), rtol=1e-6, atol=1e-7)
    want_ids = oracle.predict(loaded, X, INFER_LEAF_ID, precision)
    for storage in ("dense", "sparse"):
        fi = ForestInference.load(str(path), precision=precision, storage=storage)
        assert fi.is_classifier and fi.n_trees == 40
        Xd = _dev(X, precision)
        np.testing.assert_allclose(fi.predict_proba(Xd).cpu().numpy(), want, **_tol(loaded, precision))
        assert np.array_equal(fi.apply(Xd).cpu().numpy().astype(np.uint32), want_ids)
        # chunk_size asks for the regular (quantised, when it exists) path on this small batch
        assert np.array_equal(fi.apply(Xd, chunk_size=4).cpu().numpy().astype(np.uint32), want_ids)


def test_optimize_picks_a_chunk_size_and_keeps_results():
    desc = random_forest_desc(91, n_trees=30, n_features=8, max_depth=6, postproc="sigmoid")
    fi = ForestInference.load_from_treelite_model(desc, is_classifier=True)
    X = _dev(random_rows(12, 2000, 8, np.float32), "single")
    before = fi.predict_proba(X).cpu().numpy()
    best = fi.optimize(batch_size=512, unique_batches=2, timeout=0.05)
    assert best in (1, 2, 4, 8, 16, 32) and fi.default_chunk_size == best
    after = fi.predict_proba(X).cpu().numpy()
    # another chunk size means another tile shape and summation order: same tolerance as parity
    np.testing.assert_allclose(after, before, rtol=1e-5, atol=1e-6)


def test_optimize_sweeps_node_orders_for_the_plain_sparse_kernel():
    desc = random_forest_desc(92, n_trees=40, n_features=8, max_depth=11, p_leaf=0.2)
    X = _dev(random_rows(13, 3000, 8, np.float32), "single")
    want = oracle.predict(desc, X.cpu().numpy(), INFER_LEAF_ID, "single")
    # without a compact image the node order matters: all three are tried by default
    fi = ForestInference.load_from_treelite_model(desc, storage="sparse", compact_nodes=False,
                                                  layout="layered")
    best = fi.optimize(batch_size=1024, unique_batches=2, timeout=0.05)
    assert best in (1, 2, 4, 8, 16, 32) and fi.layout in ("depth_first", "breadth_first", "layered")
    assert fi.describe()["layout"] == {"depth_first": 0, "breadth_first": 1, "layered": 2}[fi.layout]
    assert np.array_equal(fi.apply(X).cpu().numpy().astype(np.uint32), want)
    # with it the sweep is skipped unless asked for
    fc = ForestInference.load_from_treelite_model(desc, storage="sparse")
    fc.optimize(batch_size=1024, unique_batches=2, timeout=0.05)
    assert fc.layout == "depth_first"
    fc.optimize(batch_size=1024, unique_batches=2, timeout=0.05, layouts=["breadth_first"])
    assert fc.layout == "breadth_first"
    assert np.array_equal(fc.apply(X).cpu().numpy().astype(np.uint32), want)


def test_module_level_constructor_matches_reference_call():
    # the call cuML makes: python/cuml/cuml/ensemble/randomforest_common.pyx:402-409
    from cuml_b200 import fil as nvforest

    desc, X, exp = load_golden("rfc_depth8")
    m = nvforest.load_from_treelite_model(tl_model=desc, device="gpu", layout="breadth_first",
                                          default_chunk_size=4, align_bytes=128, handle=None)
    assert "ForestInferenceClassifier" in type(m).__name__
    assert m.forest.get_dtype() == np.float32
    np.testing.assert_allclose(m.predict_proba(X), exp["proba"], rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        nvforest.load_from_treelite_model(tl_model=desc, device="cpu")


def test_more_than_2_to_31_input_elements():
    """1,000,000 x 2,150 fp32 inputs hold more than 2^31 elements; the reference runs this shape
    only to see that nothing overflows (cpp/tests/sg/rf_test.cu:908-955).  Here a sample of rows
    from the far end of the batch is also checked against the oracle."""
    torch = _torch()
    n, nf = 1_000_000, 2150
    desc = random_forest_desc(95, n_trees=10, n_features=nf, max_depth=6, n_outputs=2,
                              vector=True, average=True)
    X = torch.empty((n, nf), device="cuda:0", dtype=torch.float32)
    g = torch.Generator(device="cuda:0")
    g.manual_seed(1)
    for b in range(0, n, 100_000):
        X[b:b + 100_000] = torch.randn((100_000, nf), generator=g, device="cuda:0")
    for quantize_rows in (True, False):
        fi = ForestInference.load_from_treelite_model(desc, quantize_rows=quantize_rows)
        proba = fi.predict_proba(X)
        ids = fi.apply(X)
        idx = torch.cat([torch.arange(0, 64), torch.arange(n - 64, n)]).to("cuda:0")
        Xs = X[idx].cpu().numpy()
        np.testing.assert_allclose(proba[idx].cpu().numpy(),
                                   oracle.predict(desc, Xs, INFER_DEFAULT, "single"),
                                   rtol=1e-5, atol=1e-6)
        assert np.array_equal(ids[idx].cpu().numpy().astype(np.uint32),
                              oracle.predict(desc, Xs, INFER_LEAF_ID, "single"))
        del proba, ids
    del X
    torch.cuda.empty_cache()


def test_estimator_style_callers_against_sklearn():
    """The wrappers that use the library the way cuML's estimators do: labels, log-probabilities,
    scores, out-of-bag votes through predict_per_tree, isolation-forest scores."""
    import pickle

    from sklearn.datasets import make_classification, make_regression
    from sklearn.ensemble import IsolationForest as SkIF
    from sklearn.ensemble import RandomForestClassifier as SkRFC
    from sklearn.ensemble import RandomForestRegressor as SkRFR

    from cuml_b200.ensemble import IsolationForest, RandomForestClassifier, RandomForestRegressor

    X, y = make_classification(n_samples=1500, n_features=12, n_informative=6, n_classes=3,
                               random_state=0)
    X = X.astype(np.float32)
    y = np.array(["a", "b", "c"])[y]
    sk = SkRFC(n_estimators=25, max_depth=7, random_state=0).fit(X, y)
    m = RandomForestClassifier.from_sklearn(sk)
    proba = sk.predict_proba(X)
    np.testing.assert_allclose(m.predict_proba(X), proba, rtol=1e-5, atol=1e-6)
    top2 = np.sort(proba, axis=1)[:, -2:]
    safe = top2[:, 1] - top2[:, 0] > 1e-4
    assert np.array_equal(m.predict(X)[safe], sk.predict(X)[safe])
    with np.errstate(divide="ignore"):
        np.testing.assert_allclose(m.predict_log_proba(X), np.log(proba), rtol=1e-4, atol=1e-5)
    assert abs(m.score(X, y) - sk.score(X, y)) < 5e-3
    assert np.array_equal(m.predict(X, layout="breadth_first", default_chunk_size=2)[safe],
                          sk.predict(X)[safe])
    m2 = pickle.loads(pickle.dumps(m))
    np.testing.assert_allclose(m2.predict_proba(X), proba, rtol=1e-5, atol=1e-6)
    # out-of-bag: with no row in any bag the OOB vote is the plain forest average
    oob = m.oob_decision_function(X, np.zeros((25, X.shape[0]), bool))
    np.testing.assert_allclose(oob, proba, rtol=1e-5, atol=1e-6)

    Xr, yr = make_regression(n_samples=1200, n_features=10, noise=0.1, random_state=0)
    Xr = Xr.astype(np.float32)
    skr = SkRFR(n_estimators=20, max_depth=9, random_state=0).fit(Xr, yr)
    r = RandomForestRegressor.from_sklearn(skr, precision="double")
    pred = r.predict(Xr.astype(np.float64))
    assert pred.ndim == 1
    np.testing.assert_allclose(pred, skr.predict(Xr), rtol=1e-10, atol=1e-10)
    assert abs(r.score(Xr.astype(np.float64), yr) - skr.score(Xr, yr)) < 1e-9

    rng = np.random.default_rng(0)
    Xi = rng.standard_normal((800, 6)).astype(np.float32)
    Xi[:20] += 6.0
    ski = SkIF(n_estimators=50, random_state=0).fit(Xi)
    iso = IsolationForest.from_sklearn(ski)
    # the reference's own boundary test uses rtol=1e-5, atol=1e-6
    # (python/cuml/tests/test_isolation_forest.py:751-762)
    np.testing.assert_allclose(iso.score_samples(Xi), ski.score_samples(Xi), rtol=1e-5, atol=1e-6)
    d = ski.decision_function(Xi)
    safe = np.abs(d) > 1e-5
    assert np.array_equal(iso.predict(Xi)[safe], ski.predict(Xi)[safe])
    one = iso.score_samples(Xi[:1])  # single-sample edge case (test_isolation_forest.py:765-776)
    np.testing.assert_allclose(one, ski.score_samples(Xi[:1]), rtol=1e-5, atol=1e-6)


def test_graph_replay_of_a_small_batch():
    """A small batch recorded once as a CUDA graph and replayed gives the same answers as direct
    calls, for new inputs written into the graph's static buffer."""
    torch = _torch()
    desc = synthetic_complete_forest(200, 6, 32, seed=11)
    fi = ForestInference.load_from_treelite_model(desc)
    graphed = fi.capture_graph(512, "predict_proba")
    for seed in (1, 2, 3):
        X = torch.as_tensor(random_rows(seed, 512, 32, np.float32, nan_frac=0.02), device="cuda:0")
        got = graphed(X).clone()
        want = fi.predict_proba(X)
        torch.cuda.synchronize()
        np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=1e-6, atol=1e-7)
    with pytest.raises(ValueError):
        graphed(torch.zeros((100, 32), device="cuda:0"))


@pytest.mark.parametrize("n_trees,depth,n_classes", [(300, 5, 3), (2100, 4, 1), (40, 3, 1),
                                                     (30, 12, 1), (1, 2, 1), (37, 10, 1)])
def test_quantised_traversal_kernel_variants(n_trees, depth, n_classes):
    """Every variant of the traversal over rank-quantised rows: top nodes in the parameter block
    (up to 2048 trees of depth 4..10), the same depth-specialised kernel without them (more
    trees), the generic-depth kernel (depth 3 and 12), partial tree batches, NaN and NaN-free
    tiles, one and several classes."""
    kw = dict(n_classes=n_classes) if n_classes > 1 else {}
    desc = synthetic_complete_forest(n_trees, depth, 24, seed=40 + depth, **kw)
    rng = np.random.default_rng(41)
    n = 6000
    X = rng.standard_normal((n, 24)).astype(np.float32)
    X[:3000][rng.random((3000, 24)) < 0.05] = np.nan  # the second half stays NaN-free
    fi = ForestInference.load_from_treelite_model(desc)
    assert fi.describe()["row_quantization"] == 1
    Xd = _dev(X, "single")
    from cuml_b200.fil import _lib

    lib = _lib.load()
    try:
        # q_pair = 1 forces the walk that fetches both children of a node ahead of the test (the
        # variant for launch shapes with few walks in flight), 0 forbids it
        for pair, shape in ((0, None), (1, None), (1, (128, 2, 2, 2, 1)), (1, (64, 3, 4, 2, 1)),
                            (1, (32, 1, 1, 2, 1))):
            lib.b2fil_set_tuning(b"q_pair", pair)
            for key, v in zip((b"q_R", b"q_G", b"q_NT", b"q_S", b"q_K"), shape or (0, 0, 0, 0, 0)):
                lib.b2fil_set_tuning(key, v)
            for chunk_size in (8, 2):  # 256-row and 64-row tiles of the quantised path
                raw = fi._run(Xd, INFER_DEFAULT, chunk_size).cpu().numpy()
                if pair and (shape or n_trees != 2100):
                    assert "dense_q_pair_kernel" in _lib.last_variant() or shape is None
                np.testing.assert_allclose(raw, oracle.predict(desc, X, INFER_DEFAULT, "single"),
                                           **_tol(desc, "single"))
                ids = fi.apply(Xd, chunk_size=chunk_size).cpu().numpy()
                assert np.array_equal(ids.astype(np.uint32),
                                      oracle.predict(desc, X, INFER_LEAF_ID, "single"))
    finally:
        lib.b2fil_set_tuning(b"q_pair", -1)
        lib.b2fil_set_tuning(b"q_R", 0)


@pytest.mark.parametrize("n_trees,depth,n_classes,n_features",
                         [(37, 10, 1, 24), (50, 9, 1, 600), (45, 10, 3, 24), (7, 9, 1, 24)])
def test_quantised_walk_with_leaf_payloads_in_global_memory(n_trees, depth, n_classes, n_features):
    """Depth 9 and 10, fp32 scalar leaves: the variant whose stages hold only the test nodes and
    whose walks fetch the leaf payload from the forest image, consumed one sub-batch later.
    Forced on (q_leafg = 1) with two, three and four trees in flight, partial last sub-batches,
    several classes, tiles with and without NaN; and chosen automatically where it puts more
    walks in flight (600 features: the row tile leaves room for few whole trees)."""
    kw = dict(n_classes=n_classes) if n_classes > 1 else {}
    desc = synthetic_complete_forest(n_trees, depth, n_features, seed=60 + depth, **kw)
    rng = np.random.default_rng(61)
    n = 5000
    X = rng.standard_normal((n, n_features)).astype(np.float32)
    X[:2500][rng.random((2500, n_features)) < 0.05] = np.nan
    fi = ForestInference.load_from_treelite_model(desc)
    assert fi.describe()["row_quantization"] == 1
    Xd = _dev(X, "single")
    want = oracle.predict(desc, X, INFER_DEFAULT, "single")
    from cuml_b200.fil import _lib

    lib = _lib.load()
    try:
        if n_features == 600:
            raw = fi._run(Xd, INFER_DEFAULT, 4).cpu().numpy()
            assert "dense_q_leafg_kernel" in _lib.last_variant()
            np.testing.assert_allclose(raw, want, **_tol(desc, "single"))
        lib.b2fil_set_tuning(b"q_leafg", 1)
        for shape in (None, (128, 2, 2, 2, 1), (64, 3, 3, 2, 1), (32, 2, 4, 2, 2), (128, 1, 2, 3, 1)):
            if shape and n_features == 600 and shape[0] > 64:
                continue  # a 128-row tile of 600 features leaves no room for these stages
            for key, v in zip((b"q_R", b"q_G", b"q_NT", b"q_S", b"q_K"), shape or (0, 0, 0, 0, 0)):
                lib.b2fil_set_tuning(key, v)
            raw = fi._run(Xd, INFER_DEFAULT, 4).cpu().numpy()
            assert "dense_q_leafg_kernel" in _lib.last_variant(), _lib.last_variant()
            np.testing.assert_allclose(raw, want, **_tol(desc, "single"))
        lib.b2fil_set_tuning(b"q_leafg", 0)
        lib.b2fil_set_tuning(b"q_R", 0)
        raw = fi._run(Xd, INFER_DEFAULT, 4).cpu().numpy()
        assert "dense_q_leafg_kernel" not in _lib.last_variant()
        np.testing.assert_allclose(raw, want, **_tol(desc, "single"))
        fi.check_status()
    finally:
        lib.b2fil_set_tuning(b"q_leafg", -1)
        lib.b2fil_set_tuning(b"q_R", 0)


@pytest.mark.parametrize("precision", ["single", "double"])
def test_per_tree_outputs_wide_and_narrow_stores(precision):
    """Leaf ids and per-tree values leave the quantised traversal as 16-byte stores when a row's
    four outputs are contiguous and aligned, and as scalar stores otherwise: a tree count that is
    a multiple of four (wide), one that is not, an output buffer that starts 4 bytes off a
    16-byte boundary, and a multi-class forest whose trees are stored class by class."""
    torch = _torch()
    rng = np.random.default_rng(50)
    n = 5000
    X = rng.standard_normal((n, 16)).astype(np.float32)
    X[rng.random((n, 16)) < 0.02] = np.nan
    for n_trees, n_classes in ((24, 1), (23, 1), (24, 3)):
        kw = dict(n_classes=n_classes) if n_classes > 1 else {}
        desc = synthetic_complete_forest(n_trees, 5, 16, seed=51 + n_trees, **kw)
        fi = ForestInference.load_from_treelite_model(desc, precision=precision)
        Xd = _dev(X, precision)
        want_ids = oracle.predict(desc, X, INFER_LEAF_ID, precision)
        want_pt = oracle.predict(desc, X, INFER_PER_TREE, precision)
        ids = fi.apply(Xd, chunk_size=8).cpu().numpy()
        assert np.array_equal(ids.astype(np.uint32), want_ids)
        pt = fi.predict_per_tree(Xd, chunk_size=8).cpu().numpy()
        assert np.array_equal(pt, want_pt)
        # output buffer one element past an aligned address
        buf = torch.zeros(n * n_trees + 1, device="cuda:0", dtype=torch.int32)
        view = buf[1:].view(n, n_trees)
        fi.apply(Xd, preds=view, chunk_size=8)
        assert np.array_equal(view.cpu().numpy().astype(np.uint32), want_ids)
        assert int(buf[0]) == 0
    # the walk over the compact image of a sparse forest stores the same way
    from cuml_b200.fil import _lib

    for n_trees in (24, 23):
        desc = random_forest_desc(70 + n_trees, n_trees=n_trees, n_features=16, max_depth=12,
                                  p_leaf=0.15)
        fi = ForestInference.load_from_treelite_model(desc, precision=precision, storage="sparse")
        Xd = _dev(X, precision)
        want_ids = oracle.predict(desc, X, INFER_LEAF_ID, precision)
        want_pt = oracle.predict(desc, X, INFER_PER_TREE, precision)
        assert np.array_equal(fi.apply(Xd).cpu().numpy().astype(np.uint32), want_ids)
        assert "sparse_compact_kernel" in _lib.last_variant()
        assert np.array_equal(fi.predict_per_tree(Xd).cpu().numpy(), want_pt)
        buf = torch.zeros(n * n_trees + 1, device="cuda:0", dtype=torch.int32)
        view = buf[1:].view(n, n_trees)
        fi.apply(Xd, preds=view)
        assert np.array_equal(view.cpu().numpy().astype(np.uint32), want_ids)
        assert int(buf[0]) == 0
        real = torch.float32 if precision == "single" else torch.float64
        buf = torch.zeros(n * n_trees + 1, device="cuda:0", dtype=real)
        view = buf[1:].view(n, n_trees)
        fi.predict_per_tree(Xd, preds=view)
        assert np.array_equal(view.cpu().numpy(), want_pt)
        assert float(buf[0]) == 0.0
