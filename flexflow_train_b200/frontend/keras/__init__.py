"""Keras-compatible surface: ``layers``, ``models``, ``optimizers``, ``losses``, ``metrics``, ``callbacks``, ``initializers``,
``regularizers``, ``backend``, ``utils``, ``preprocessing``, ``datasets``."""
from . import backend, callbacks, datasets, initializers, layers, losses, metrics, models, optimizers, preprocessing, regularizers, utils  # noqa: F401
from .layers import Input  # noqa: F401
from .models import Model, Sequential  # noqa: F401
