"""Enumerations of the Python frontend.

Member names follow the legacy Python API (bindings/python/old/flexflow/type.py) so existing model scripts keep
reading naturally; the *values* are the strings the IR uses, so no translation table is needed between the
frontend and the compiler core.
"""
from __future__ import annotations

from enum import Enum


class ActiMode(Enum):
    AC_MODE_NONE = None
    AC_MODE_RELU = "RELU"
    AC_MODE_SIGMOID = "SIGMOID"
    AC_MODE_TANH = "TANH"
    AC_MODE_GELU = "GELU"


class RegularizerMode(Enum):
    REG_MODE_NONE = "none"
    REG_MODE_L1 = "l1"
    REG_MODE_L2 = "l2"


class AggrMode(Enum):
    AGGR_MODE_NONE = "NONE"
    AGGR_MODE_SUM = "SUM"
    AGGR_MODE_AVG = "AVG"


class PoolType(Enum):
    POOL_MAX = "MAX"
    POOL_AVG = "AVG"


class DataType(Enum):
    DT_BOOLEAN = "BOOL"
    DT_INT32 = "INT32"
    DT_INT64 = "INT64"
    DT_HALF = "HALF"
    DT_FLOAT = "FLOAT"
    DT_DOUBLE = "DOUBLE"
    DT_NONE = "NONE"


class LossType(Enum):
    LOSS_CATEGORICAL_CROSSENTROPY = "categorical_crossentropy"
    LOSS_SPARSE_CATEGORICAL_CROSSENTROPY = "sparse_categorical_crossentropy"
    LOSS_MEAN_SQUARED_ERROR_AVG_REDUCE = "mean_squared_error_avg_reduce"
    LOSS_MEAN_SQUARED_ERROR_SUM_REDUCE = "mean_squared_error_sum_reduce"
    LOSS_IDENTITY = "identity"


class CompMode(Enum):
    TRAINING = "training"
    INFERENCE = "inference"


class ParameterSyncType(Enum):
    NONE = "none"
    PS = "ps"        # accepted for source compatibility; gradients are always reduced over NVLink
    NCCL = "nccl"


class MetricsType(Enum):
    METRICS_ACCURACY = "accuracy"
    METRICS_CATEGORICAL_CROSSENTROPY = "categorical_crossentropy"
    METRICS_SPARSE_CATEGORICAL_CROSSENTROPY = "sparse_categorical_crossentropy"
    METRICS_MEAN_SQUARED_ERROR = "mean_squared_error"
    METRICS_ROOT_MEAN_SQUARED_ERROR = "root_mean_squared_error"
    METRICS_MEAN_ABSOLUTE_ERROR = "mean_absolute_error"


class OpType(Enum):
    """Operator kinds the importers emit (the text IR of the torch.fx importer stores these names)."""
    CONV2D = "CONV2D"
    EMBEDDING = "EMBEDDING"
    POOL2D = "POOL2D"
    LINEAR = "LINEAR"
    SOFTMAX = "SOFTMAX"
    CONCAT = "CONCAT"
    FLAT = "FLAT"
    BATCH_NORM = "BATCHNORM"
    LAYER_NORM = "LAYERNORM"
    RELU = "RELU"
    SIGMOID = "SIGMOID"
    TANH = "TANH"
    ELU = "ELU"
    GELU = "GELU"
    IDENTITY = "IDENTITY"
    DROPOUT = "DROPOUT"
    BATCH_MATMUL = "BATCHMATMUL"
    SPLIT = "SPLIT"
    RESHAPE = "RESHAPE"
    TRANSPOSE = "TRANSPOSE"
    REVERSE = "REVERSE"
    GATHER = "GATHER"
    EXP = "EXP"
    SIN = "SIN"
    COS = "COS"
    RSQRT = "RSQRT"
    POW = "POW"
    ADD = "EW_ADD"
    SUBTRACT = "EW_SUB"
    MULTIPLY = "EW_MUL"
    DIVIDE = "EW_DIV"
    MAX = "EW_MAX"
    MIN = "EW_MIN"
    SCALAR_MULTIPLY = "SCALAR_MULTIPLY"
    SCALAR_ADD = "SCALAR_ADD"
    SCALAR_SUB = "SCALAR_SUB"
    SCALAR_TRUEDIV = "SCALAR_TRUE_DIV"
    SCALAR_FLOORDIV = "SCALAR_FLOOR_DIV"
    REDUCE_SUM = "REDUCE_SUM"
    MEAN = "REDUCE_MEAN"
    MULTIHEAD_ATTENTION = "MULTIHEAD_ATTENTION"
    INPUT = "INPUT"
    OUTPUT = "OUTPUT"
    GETITEM = "GETITEM"
    GETATTR = "GETATTR"
    ATTRIBUTE = "ATTRIBUTE"
    EXPAND = "EXPAND"
    PERMUTE = "PERMUTE"
    VIEW = "VIEW"
    TO = "TO"
    UNSQUEEZE = "UNSQUEEZE"
    FLOAT = "FLOAT"
    TYPE_AS = "TYPE_AS"
    CONTIGUOUS = "CONTIGUOUS"
    LAYER_NORM_T5 = "T5_LAYERNORM"


def enum_value(v):
    """Accept an enum member or its raw value."""
    return v.value if isinstance(v, Enum) else v
