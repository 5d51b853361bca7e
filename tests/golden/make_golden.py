"""Generates the golden fixtures of this directory with scikit-learn (an implementation that is
independent of both the CPU oracle and the CUDA kernels).

    python tests/golden/make_golden.py

Each .npz holds: the forest description imported from the fitted model, test rows, and what
scikit-learn itself returns for them (predict_proba / predict / apply).  Shapes follow the
benchmark configurations at reduced size: a depth-8 random-forest classifier on 32 fp32 features
(2 classes), an unpruned depth-20 random-forest regressor on 64 fp64 features, a 3-class gradient
boosted classifier, and a forest trained on data with missing values (per-node default direction).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from sklearn.datasets import make_classification, make_regression  # noqa: E402
from sklearn.ensemble import (GradientBoostingClassifier, RandomForestClassifier,  # noqa: E402
                              RandomForestRegressor)

from cuml_b200.fil.importers import from_sklearn  # noqa: E402


def save(name, model, X, **expected):
    d = {("desc_" + k): v for k, v in from_sklearn(model).to_dict().items() if v is not None}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), X=X, **d, **expected)
    print(name, {k: v.shape for k, v in expected.items()})


def main():
    # depth-8 random-forest classifier, 32 fp32 features, 2 classes (benchmark config 1, smaller)
    X, y = make_classification(n_samples=4000, n_features=32, n_informative=16, n_classes=2,
                               random_state=0)
    X = X.astype(np.float32)
    m = RandomForestClassifier(n_estimators=20, max_depth=8, random_state=0).fit(X, y)
    Xt = make_classification(n_samples=3000, n_features=32, n_informative=16, n_classes=2,
                             random_state=1)[0].astype(np.float32)
    save("rfc_depth8", m, Xt, proba=m.predict_proba(Xt), labels=m.predict(Xt).astype(np.int64),
         leaf_ids=m.apply(Xt).astype(np.int64))

    # unpruned random-forest regressor, 64 fp64 features (benchmark config 3, smaller); test rows
    # are fp32-representable because scikit-learn itself predicts on fp32-rounded inputs
    X, y = make_regression(n_samples=6000, n_features=64, noise=0.1, random_state=0)
    m = RandomForestRegressor(n_estimators=8, max_depth=20, min_samples_leaf=1,
                              random_state=0).fit(X, y)
    Xt = make_regression(n_samples=2000, n_features=64, noise=0.1, random_state=1)[0]
    Xt = Xt.astype(np.float32).astype(np.float64)
    save("rfr_depth20", m, Xt, values=m.predict(Xt), leaf_ids=m.apply(Xt).astype(np.int64))

    # 3-class gradient boosting: scalar leaves, one tree per class and round, softmax
    X, y = make_classification(n_samples=3000, n_features=12, n_informative=8, n_classes=3,
                               random_state=2)
    m = GradientBoostingClassifier(n_estimators=25, max_depth=4, random_state=0).fit(X, y)
    Xt = make_classification(n_samples=2000, n_features=12, n_informative=8, n_classes=3,
                             random_state=3)[0]
    Xt = Xt.astype(np.float32).astype(np.float64)
    save("gbc_3class", m, Xt, proba=m.predict_proba(Xt), labels=m.predict(Xt).astype(np.int64))

    # missing values: trees learn a per-node direction for NaN
    rng = np.random.default_rng(4)
    X, y = make_classification(n_samples=3000, n_features=10, n_informative=6, n_classes=2,
                               random_state=4)
    X = X.astype(np.float32)
    X[rng.random(X.shape) < 0.1] = np.nan
    m = RandomForestClassifier(n_estimators=12, max_depth=7, random_state=0).fit(X, y)
    Xt = make_classification(n_samples=2000, n_features=10, n_informative=6, n_classes=2,
                             random_state=5)[0].astype(np.float32)
    Xt[rng.random(Xt.shape) < 0.1] = np.nan
    save("rfc_missing", m, Xt, proba=m.predict_proba(Xt), labels=m.predict(Xt).astype(np.int64),
         leaf_ids=m.apply(Xt).astype(np.int64))


if __name__ == "__main__":
    main()
