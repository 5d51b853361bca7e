"""Estimator-style callers of the inference library, mirroring how cuML's own estimators use it.

These classes hold a fitted forest (imported from scikit-learn) and forward prediction to
`cuml_b200.fil.ForestInference` the way the reference's estimators forward to their inference
library: a cached model for the default options, a rebuilt one for non-default `layout` /
`default_chunk_size` / `align_bytes` (python/cuml/cuml/ensemble/randomforest_common.pyx:624-642),
class indices mapped to labels (randomforestclassifier.py:337-338), regressor outputs squeezed to
one dimension (randomforestregressor.py:269-275), out-of-bag scoring through `predict_per_tree`
(randomforest_common.pyx:644-702) and the isolation-forest score transform
(python/cuml/cuml/ensemble/isolation_forest.pyx:1015-1030).  Training is not part of this
library: models are fitted elsewhere and imported.
"""
from __future__ import annotations

import numpy as np

from .fil import ForestInference, from_sklearn
from .fil._desc import ForestDesc


def _to_numpy(a):
    return a if isinstance(a, np.ndarray) else a.detach().cpu().numpy()


class _ForestModel:
    _default = dict(layout="depth_first", default_chunk_size=None, align_bytes=None)

    def __init__(self, desc: ForestDesc, precision: str = "single", device_id: int = 0):
        self._desc = desc
        self._precision = precision
        self._device_id = device_id
        self._cached = None

    def _inference_model(self, layout="depth_first", default_chunk_size=None, align_bytes=None):
        opts = dict(layout=layout, default_chunk_size=default_chunk_size, align_bytes=align_bytes)
        if opts == self._default:
            if self._cached is None:
                self._cached = self.as_fil(**opts)
            return self._cached
        return self.as_fil(**opts)

    def as_fil(self, layout="depth_first", default_chunk_size=None, align_bytes=None):
        """A `ForestInference` for this model (counterpart of `as_nvforest`,
        randomforest_common.pyx:373-409)."""
        return ForestInference.load_from_treelite_model(
            self._desc, layout=layout, default_chunk_size=default_chunk_size,
            align_bytes=align_bytes, precision=self._precision, device_id=self._device_id)

    def __getstate__(self):
        st = dict(self.__dict__)
        st["_cached"] = None  # the device forest is rebuilt lazily after unpickling
        st["_desc"] = self._desc.to_dict()
        return st

    def __setstate__(self, st):
        self.__dict__.update(st)
        self._desc = ForestDesc.from_dict(st["_desc"])


class RandomForestClassifier(_ForestModel):
    """Inference side of a random-forest classifier."""

    def __init__(self, desc, classes, precision="single", device_id=0):
        super().__init__(desc, precision, device_id)
        self.classes_ = np.asarray(classes)
        self.n_classes_ = len(self.classes_)

    @classmethod
    def from_sklearn(cls, model, precision="single", device_id=0):
        return cls(from_sklearn(model), model.classes_, precision, device_id)

    def predict_proba(self, X, *, layout="depth_first", default_chunk_size=None, align_bytes=None):
        return self._inference_model(layout, default_chunk_size, align_bytes).predict_proba(X)

    def predict_log_proba(self, X, **kw):
        out = self.predict_proba(X, **kw)
        return np.log(out) if isinstance(out, np.ndarray) else out.log()

    def predict(self, X, *, threshold=0.5, layout="depth_first", default_chunk_size=None,
                align_bytes=None):
        idx = self._inference_model(layout, default_chunk_size, align_bytes).predict(
            X, threshold=threshold)
        return self.classes_[_to_numpy(idx).astype(np.int64)]

    def score(self, X, y, **kw):
        return float(np.mean(self.predict(X, **kw) == np.asarray(y)))

    def oob_decision_function(self, X, in_bag_masks):
        """Average the per-tree class votes of the trees that did NOT see each row
        (`in_bag_masks[t, i]` true when row i was in tree t's bootstrap sample)."""
        per_tree = _to_numpy(self._inference_model().predict_per_tree(X))  # (n, trees, classes)
        out_of_bag = ~np.asarray(in_bag_masks, bool).T  # (n, trees)
        votes = (per_tree * out_of_bag[:, :, None]).sum(axis=1)
        count = out_of_bag.sum(axis=1, keepdims=True)
        return votes / np.where(count == 0, 1, count)


class RandomForestRegressor(_ForestModel):
    """Inference side of a random-forest regressor."""

    @classmethod
    def from_sklearn(cls, model, precision="single", device_id=0):
        return cls(from_sklearn(model), precision, device_id)

    def predict(self, X, *, layout="depth_first", default_chunk_size=None, align_bytes=None):
        out = self._inference_model(layout, default_chunk_size, align_bytes).predict(X)
        return out.reshape(-1) if out.ndim == 2 and out.shape[1] == 1 else out

    def score(self, X, y, **kw):
        pred = _to_numpy(self.predict(X, **kw)).astype(np.float64)
        y = np.asarray(y, np.float64)
        ss_res = float(((y - pred) ** 2).sum())
        ss_tot = float(((y - y.mean()) ** 2).sum())
        return 1.0 - ss_res / ss_tot if ss_tot > 0 else 0.0

    def oob_prediction(self, X, in_bag_masks):
        per_tree = _to_numpy(self._inference_model().predict_per_tree(X))  # (n, trees)
        out_of_bag = ~np.asarray(in_bag_masks, bool).T
        count = out_of_bag.sum(axis=1)
        return (per_tree * out_of_bag).sum(axis=1) / np.where(count == 0, 1, count)


class IsolationForest(_ForestModel):
    """Scoring side of an isolation forest: the forest's average path length h is turned into the
    anomaly score -2^(-h / c) with c the normalisation constant of the training sample size."""

    def __init__(self, desc, c_normalization, offset=0.0, precision="single", device_id=0):
        super().__init__(desc, precision, device_id)
        self._c_normalization = float(c_normalization)
        self.offset_ = float(offset)

    @classmethod
    def from_sklearn(cls, model, precision="single", device_id=0):
        from sklearn.ensemble._iforest import _average_path_length

        c = float(_average_path_length(np.asarray([model.max_samples_]))[0])
        return cls(from_sklearn(model), c, model.offset_, precision, device_id)

    def score_samples(self, X, **kw):
        h = self._inference_model(**kw).predict(X)
        h = h.reshape(-1) if h.ndim == 2 else h
        if self._c_normalization <= 0:
            return (h * 0) - 0.5
        return -(2.0 ** (-h / self._c_normalization))

    def decision_function(self, X, **kw):
        return self.score_samples(X, **kw) - self.offset_

    def predict(self, X, **kw):
        d = _to_numpy(self.decision_function(X, **kw))
        return np.where(d < 0, -1, 1)
