"""Keras-compatible surface: ``layers``, ``models``, ``optimizers``, ``losses``, ``metrics``, ``callbacks``."""
from . import callbacks, layers, losses, metrics, models, optimizers  # noqa: F401
from .layers import Input  # noqa: F401
from .models import Model, Sequential  # noqa: F401
