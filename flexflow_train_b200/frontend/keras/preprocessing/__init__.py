"""Keras preprocessing helpers (bindings/python/old/flexflow/keras/preprocessing)."""
from . import sequence, text  # noqa: F401
