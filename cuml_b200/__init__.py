"""cuml_b200: B200-native batched tree-ensemble prediction behind the cuml.fil interface."""
from . import fil  # noqa: F401

__version__ = "0.1.0"
