"""User-facing model frontends: the layer API (``FFModel``), the PyTorch (torch.fx) importer, the ONNX importer
and the Keras-compatible classes."""
from ..config_schema import FFConfig  # noqa: F401
from .ffmodel import (AdamOptimizer, FFModel, GlorotUniformInitializer, NormInitializer, SGDOptimizer, SingleDataLoader,  # noqa: F401
                      Tensor, UniformInitializer, ZeroInitializer)
from .dataloader import DataLoader  # noqa: F401
from .types import (ActiMode, AggrMode, CompMode, DataType, LossType, MetricsType, OpType, ParameterSyncType, PoolType,  # noqa: F401
                    RegularizerMode)
