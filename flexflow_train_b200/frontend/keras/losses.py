"""Keras-style loss identifiers (bindings/python/old/flexflow/keras/losses.py)."""
from ..types import LossType


class Loss:
    type = None

    def __init__(self, name=None):
        self.name = name


class CategoricalCrossentropy(Loss):
    type = LossType.LOSS_CATEGORICAL_CROSSENTROPY


class SparseCategoricalCrossentropy(Loss):
    type = LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY


class MeanSquaredError(Loss):
    type = LossType.LOSS_MEAN_SQUARED_ERROR_AVG_REDUCE


class Identity(Loss):
    type = LossType.LOSS_IDENTITY


_BY_NAME = {"categorical_crossentropy": LossType.LOSS_CATEGORICAL_CROSSENTROPY,
            "sparse_categorical_crossentropy": LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY,
            "mean_squared_error": LossType.LOSS_MEAN_SQUARED_ERROR_AVG_REDUCE, "mse": LossType.LOSS_MEAN_SQUARED_ERROR_AVG_REDUCE,
            "identity": LossType.LOSS_IDENTITY}


def get(identifier) -> LossType:
    if isinstance(identifier, LossType):
        return identifier
    if isinstance(identifier, Loss):
        return identifier.type
    return _BY_NAME[str(identifier).lower()]
