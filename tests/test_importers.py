"""Model-file importers on the CPU: every importer must yield a description on which the oracle
reproduces a hand-computed or independently computed answer.  XGBoost and LightGBM themselves are
not installed, so their files are written by hand here following the published formats."""
import json

import numpy as np
import pytest

from cuml_b200.fil._desc import INFER_DEFAULT, INFER_LEAF_ID, INFER_PROBA2, concatenate
from cuml_b200.fil.lightgbm_txt import from_lightgbm_text
from cuml_b200.fil.loaders import load_desc, load_file, save_desc, to_forest_desc
from cuml_b200.fil.treelite_json import from_treelite_json, to_treelite_json
from cuml_b200.fil.xgboost_json import from_xgboost_json
from oracle import oracle
from tests.helpers import load_golden, random_forest_desc, random_rows


@pytest.mark.parametrize("kw", [dict(), dict(categorical=True, mixed_ops=True),
                                dict(n_outputs=3, vector=True, average=True),
                                dict(n_outputs=4, postproc="softmax", base=True)])
def test_treelite_json_round_trip(kw):
    desc = random_forest_desc(5, n_trees=6, max_depth=5, **kw)
    dump = to_treelite_json(desc)
    back = from_treelite_json(json.loads(json.dumps(dump)))
    X = random_rows(1, 300, desc.n_features, np.float32, categories=22)
    for kind in (INFER_LEAF_ID, INFER_DEFAULT):
        assert np.array_equal(oracle.predict(desc, X, kind, "single"),
                              oracle.predict(back, X, kind, "single"))
    # the object form: anything with dump_as_json() is accepted like a treelite.Model
    class FakeTreeliteModel:
        def dump_as_json(self, pretty_print=False):
            return json.dumps(dump)

    again = to_forest_desc(FakeTreeliteModel())
    assert np.array_equal(oracle.predict(again, X, INFER_LEAF_ID, "single"),
                          oracle.predict(desc, X, INFER_LEAF_ID, "single"))


def test_treelite_json_fields_of_a_reference_dump():
    # shape of a one-node tree as the reference's own test prints it
    # (python/cuml/tests/test_random_forest.py:1185-1192)
    model = {"num_feature": 3, "num_class": [1], "leaf_vector_shape": [1, 1],
             "average_tree_output": True, "postprocessor": "identity", "base_scores": [0.0],
             "trees": [{"nodes": [{"node_id": 0, "leaf_value": 1.0, "data_count": 5}]}]}
    desc = from_treelite_json(model)
    out = oracle.predict(desc, np.zeros((2, 3), np.float32), INFER_DEFAULT, "single")
    assert np.array_equal(out, np.ones((2, 1), np.float32))


def _xgb_model(objective="binary:logistic", num_class=0):
    # two stumps: tree 0 splits feature 0 at 0.5 (missing -> left), tree 1 is categorical on
    # feature 1 with categories {1, 3} going right (missing -> right)
    t0 = {"left_children": [1, -1, -1], "right_children": [2, -1, -1], "split_indices": [0, 0, 0],
          "split_conditions": [0.5, -0.2, 0.3], "default_left": [1, 0, 0], "split_type": [0, 0, 0],
          "categories": [], "categories_nodes": [], "categories_segments": [],
          "categories_sizes": [], "base_weights": [0, -0.2, 0.3]}
    t1 = {"left_children": [1, -1, -1], "right_children": [2, -1, -1], "split_indices": [1, 0, 0],
          "split_conditions": [0.0, 0.1, -0.4], "default_left": [0, 0, 0], "split_type": [1, 0, 0],
          "categories": [1, 3], "categories_nodes": [0], "categories_segments": [0],
          "categories_sizes": [2], "base_weights": [0, 0.1, -0.4]}
    return {"learner": {"learner_model_param": {"num_feature": "2", "num_class": str(num_class),
                                                "base_score": "5E-1"},
                        "objective": {"name": objective},
                        "gradient_booster": {"name": "gbtree",
                                             "model": {"trees": [t0, t1], "tree_info": [0, 0]}}}}


def test_xgboost_json_binary_logistic():
    desc = from_xgboost_json(_xgb_model())
    X = np.array([[0.4, 1.0], [0.5, 2.0], [np.nan, 3.0], [0.7, np.nan], [0.49, 3.9]], np.float32)
    margin = np.array([-0.2 - 0.4, 0.3 + 0.1, -0.2 - 0.4, 0.3 - 0.4, -0.2 - 0.4])
    want = 1 / (1 + np.exp(-margin))
    got = oracle.predict(desc, X, INFER_PROBA2, "single")
    np.testing.assert_allclose(got[:, 1], want, rtol=1e-6)
    ids = oracle.predict(desc, X, INFER_LEAF_ID, "single")
    assert ids.tolist() == [[1, 2], [2, 1], [1, 2], [2, 2], [1, 2]]


def test_xgboost_json_regression_base_score_and_file(tmp_path):
    m = _xgb_model("reg:squarederror")
    p = tmp_path / "model.json"
    p.write_text(json.dumps(m))
    desc = load_file(str(p))
    X = np.array([[0.0, 0.0]], np.float32)
    np.testing.assert_allclose(oracle.predict(desc, X, INFER_DEFAULT, "single")[0, 0],
                               0.5 - 0.2 + 0.1, rtol=1e-6)


LGBM = """tree
version=v3
num_class=1
num_tree_per_iteration=1
label_index=0
max_feature_idx=2
objective=binary sigmoid:1
feature_names=a b c
feature_infos=[-1:1] [-1:1] 0:1:2:3

Tree=0
num_leaves=3
num_cat=0
split_feature=0 1
split_gain=1 1
threshold=0.5 -0.25
decision_type=2 8
left_child=1 -1
right_child=-3 -2
leaf_value=0.1 0.2 -0.3
leaf_weight=1 1 1
leaf_count=1 1 1
internal_value=0 0
internal_weight=0 0
internal_count=3 2
shrinkage=1

Tree=1
num_leaves=2
num_cat=1
split_feature=2
split_gain=1
threshold=0
decision_type=1
left_child=-1
right_child=-2
leaf_value=0.5 -0.5
leaf_weight=1 1
leaf_count=1 1
internal_value=0
internal_weight=0
internal_count=2
cat_boundaries=0 1
cat_threshold=10
shrinkage=1

end of trees
"""


def test_lightgbm_text():
    # tree 0: node0 (f0 <= 0.5, default left, missing none -> NaN treated as 0.0 -> left),
    #         node1 (f1 <= -0.25, missing NaN, default right); tree 1: categories {1, 3} go left
    desc = from_lightgbm_text(LGBM)
    X = np.array([[0.4, -0.3, 1], [0.4, 0.0, 2], [0.6, 0.0, 3], [np.nan, np.nan, np.nan],
                  [0.5, -0.25, 0]], np.float64)
    margin = np.array([0.1 + 0.5, 0.2 - 0.5, -0.3 + 0.5, 0.2 - 0.5, 0.1 - 0.5])
    got = oracle.predict(desc, X, INFER_PROBA2, "double")
    np.testing.assert_allclose(got[:, 1], 1 / (1 + np.exp(-margin)), rtol=1e-12)


def test_npz_checkpoint_round_trip(tmp_path):
    desc, X, exp = load_golden("rfc_missing")
    path = str(tmp_path / "forest.npz")
    save_desc(desc, path)
    back = load_desc(path)
    assert np.array_equal(oracle.predict(back, X, INFER_LEAF_ID, "single").astype(np.int64),
                          exp["leaf_ids"])
    assert load_file(path).n_trees == desc.n_trees


def test_concatenate_forests():
    a = random_forest_desc(1, n_trees=4, n_outputs=3, vector=True, average=True)
    b = random_forest_desc(2, n_trees=5, n_outputs=3, vector=True, average=True)
    c = concatenate([a, b])
    X = random_rows(3, 100, a.n_features, np.float32)
    pa = oracle.predict(a, X, INFER_DEFAULT, "double")
    pb = oracle.predict(b, X, INFER_DEFAULT, "double")
    pc = oracle.predict(c, X, INFER_DEFAULT, "double")
    np.testing.assert_allclose(pc, (4 * pa + 5 * pb) / 9, rtol=1e-12, atol=1e-14)
    ids = oracle.predict(c, X, INFER_LEAF_ID, "double")
    assert np.array_equal(ids[:, :4], oracle.predict(a, X, INFER_LEAF_ID, "double"))
    assert np.array_equal(ids[:, 4:], oracle.predict(b, X, INFER_LEAF_ID, "double"))


def test_ubjson_round_trip_and_hand_made_bytes():
    from cuml_b200.fil import ubjson

    obj = {"a": [1, 2, 300, -70000], "b": [0.5, -1.25, 3.0], "c": "text", "d": None, "e": True,
           "f": {"g": [1, "x", 2.5, [False]], "h": 2 ** 40, "i": []}, "j": [2 ** 35, 1]}
    assert ubjson.loads(ubjson.dumps(obj)) == obj
    # bytes written by hand from the specification: {"k": [$U#i 3: 1 2 3], "s": "hi", "n": no-op,
    # "v": 2.5 (float32), "w": int16 -2}
    raw = (b"{" + b"i\x01k" + b"[$U#i\x03\x01\x02\x03" + b"i\x01s" + b"S" + b"i\x02hi" +
           b"i\x01v" + b"N" + b"d" + bytes.fromhex("40200000") + b"i\x01w" + b"I\xff\xfe" + b"}")
    assert ubjson.loads(raw) == {"k": [1, 2, 3], "s": "hi", "v": 2.5, "w": -2}
    # counted object with a common value type
    raw = b"{$i#i\x02" + b"i\x01a\x05" + b"i\x01b\xfb"
    assert ubjson.loads(raw) == {"a": 5, "b": -5}
    with pytest.raises(ValueError):
        ubjson.loads(b"[$i#i\x05\x01")  # truncated


@pytest.mark.parametrize("n_classes", [1, 3])
def test_xgboost_json_and_ubjson_files_round_trip(tmp_path, n_classes):
    from cuml_b200.fil import ubjson
    from cuml_b200.fil.xgboost_json import to_xgboost_json
    from tests.helpers import xgboost_style_desc

    desc = xgboost_style_desc(7 + n_classes, n_classes=n_classes)
    obj = to_xgboost_json(desc, "multi:softprob" if n_classes > 1 else "binary:logistic")
    pj, pu = tmp_path / "m.json", tmp_path / "m.ubj"
    pj.write_text(json.dumps(obj))
    pu.write_bytes(ubjson.dumps(obj))
    X = random_rows(5, 300, desc.n_features, np.float32, categories=22)
    want = oracle.predict(desc, X, INFER_DEFAULT, "single")
    want_ids = oracle.predict(desc, X, INFER_LEAF_ID, "single")
    for path in (pj, pu):
        back = load_file(str(path))
        assert back.n_trees == desc.n_trees and back.n_outputs == desc.n_outputs
        np.testing.assert_allclose(oracle.predict(back, X, INFER_DEFAULT, "single"), want,
                                   rtol=1e-6, atol=1e-7)
        assert np.array_equal(oracle.predict(back, X, INFER_LEAF_ID, "single"), want_ids)


@pytest.mark.parametrize("n_classes", [1, 3])
def test_lightgbm_text_file_round_trip(tmp_path, n_classes):
    from cuml_b200.fil.lightgbm_txt import to_lightgbm_text
    from tests.helpers import lightgbm_style_desc

    desc = lightgbm_style_desc(11 + n_classes, n_classes=n_classes)
    p = tmp_path / "m.txt"
    p.write_text(to_lightgbm_text(desc, f"multiclass num_class:{n_classes}" if n_classes > 1
                                  else "binary sigmoid:1.5"))
    back = load_file(str(p))
    X = random_rows(6, 300, desc.n_features, np.float64, categories=22)
    np.testing.assert_allclose(oracle.predict(back, X, INFER_DEFAULT, "double"),
                               oracle.predict(desc, X, INFER_DEFAULT, "double"),
                               rtol=1e-12, atol=1e-13)
