"""Model sources other than scikit-learn: dispatch by object type or file type."""
from __future__ import annotations

import json
import os
from typing import Optional

import numpy as np

from ._desc import ForestDesc


def to_forest_desc(model) -> ForestDesc:
    """Accept a `ForestDesc`, a Treelite-like object (`dump_as_json()`), a JSON dump (str/dict) or
    a fitted scikit-learn estimator."""
    if isinstance(model, ForestDesc):
        return model
    if hasattr(model, "dump_as_json"):
        from .treelite_json import from_treelite_json

        return from_treelite_json(json.loads(model.dump_as_json(pretty_print=False)))
    if isinstance(model, dict):
        from .treelite_json import from_treelite_json

        return from_treelite_json(model)
    if isinstance(model, (str, bytes)):
        from .treelite_json import from_treelite_json

        return from_treelite_json(json.loads(model))
    if hasattr(model, "n_features_in_"):
        from .importers import from_sklearn

        return from_sklearn(model)
    raise TypeError(f"cannot import a model of type {type(model).__name__}")


def save_desc(desc: ForestDesc, path: str) -> None:
    """Write a forest description as one .npz file (the checkpoint format of this library)."""
    d = {k: v for k, v in desc.to_dict().items() if v is not None}
    np.savez_compressed(path, **d)


def load_desc(path: str) -> ForestDesc:
    with np.load(path, allow_pickle=False) as z:
        d = {k: z[k] for k in z.files}
    out = {}
    for k in ForestDesc._SCALARS:
        v = d[k]
        out[k] = v.item() if hasattr(v, "item") else v
    for k in ForestDesc._ARRAYS:
        out[k] = d.get(k)
    out["postproc"] = str(out["postproc"])
    out["native_precision"] = str(out["native_precision"])
    return ForestDesc(**out)


def load_file(path: str, model_type: Optional[str] = None) -> ForestDesc:
    if model_type is None:
        ext = os.path.splitext(path)[1].lower()
        model_type = {".json": "xgboost_json", ".ubj": "xgboost_ubjson", ".txt": "lightgbm",
                      ".npz": "b2fil_npz", ".model": "lightgbm"}.get(ext)
        if model_type == "xgboost_json":
            with open(path) as fh:
                head = json.load(fh)
            if "trees" in head and "learner" not in head:
                from .treelite_json import from_treelite_json

                return from_treelite_json(head)
    if model_type == "b2fil_npz":
        return load_desc(path)
    if model_type == "treelite_json":
        from .treelite_json import from_treelite_json

        with open(path) as fh:
            return from_treelite_json(json.load(fh))
    if model_type in ("xgboost_json", "xgboost"):
        from .xgboost_json import from_xgboost_json

        with open(path) as fh:
            return from_xgboost_json(json.load(fh))
    if model_type in ("xgboost_ubjson", "xgboost_ubj"):
        from . import ubjson
        from .xgboost_json import from_xgboost_json

        with open(path, "rb") as fh:
            return from_xgboost_json(ubjson.loads(fh.read()))
    if model_type in ("lightgbm", "lightgbm_txt"):
        from .lightgbm_txt import from_lightgbm_text

        with open(path) as fh:
            return from_lightgbm_text(fh.read())
    raise ValueError(f"unknown model_type {model_type!r} for {path}")
