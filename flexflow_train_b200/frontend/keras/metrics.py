"""Keras-style metric identifiers (bindings/python/old/flexflow/keras/metrics.py)."""
from ..types import MetricsType


class Metric:
    type = None


class Accuracy(Metric):
    type = MetricsType.METRICS_ACCURACY


class CategoricalCrossentropy(Metric):
    type = MetricsType.METRICS_CATEGORICAL_CROSSENTROPY


class SparseCategoricalCrossentropy(Metric):
    type = MetricsType.METRICS_SPARSE_CATEGORICAL_CROSSENTROPY


class MeanSquaredError(Metric):
    type = MetricsType.METRICS_MEAN_SQUARED_ERROR


class RootMeanSquaredError(Metric):
    type = MetricsType.METRICS_ROOT_MEAN_SQUARED_ERROR


class MeanAbsoluteError(Metric):
    type = MetricsType.METRICS_MEAN_ABSOLUTE_ERROR


_BY_NAME = {"accuracy": MetricsType.METRICS_ACCURACY, "acc": MetricsType.METRICS_ACCURACY,
            "categorical_crossentropy": MetricsType.METRICS_CATEGORICAL_CROSSENTROPY,
            "sparse_categorical_crossentropy": MetricsType.METRICS_SPARSE_CATEGORICAL_CROSSENTROPY,
            "mean_squared_error": MetricsType.METRICS_MEAN_SQUARED_ERROR, "mse": MetricsType.METRICS_MEAN_SQUARED_ERROR,
            "root_mean_squared_error": MetricsType.METRICS_ROOT_MEAN_SQUARED_ERROR,
            "mean_absolute_error": MetricsType.METRICS_MEAN_ABSOLUTE_ERROR, "mae": MetricsType.METRICS_MEAN_ABSOLUTE_ERROR}


def get(identifier) -> MetricsType:
    if isinstance(identifier, MetricsType):
        return identifier
    if isinstance(identifier, Metric):
        return identifier.type
    return _BY_NAME[str(identifier).lower()]
