"""B200 forest inference: drop-in for the `cuml.fil.ForestInference` surface."""
from ._desc import ForestDesc, concatenate
from .forest_inference import (ForestInference, ForestInferenceClassifier,
                               ForestInferenceRegressor, load_from_treelite_model)
from .importers import from_sklearn, synthetic_complete_forest

__all__ = ["ForestInference", "ForestInferenceClassifier", "ForestInferenceRegressor",
           "ForestDesc", "concatenate", "from_sklearn", "synthetic_complete_forest",
           "load_from_treelite_model"]
