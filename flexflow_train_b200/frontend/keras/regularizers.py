"""Keras-style weight regularizers (bindings/python/old/flexflow/keras/regularizers.py).  ``L2(l)`` on a Dense kernel is
the per-layer form of weight decay: the value is recorded on the layer; the optimizers apply one decay to all weights
(``weight_decay``), so a model whose layers all carry the same L2 factor trains identically with that factor as the
optimizer's decay."""
from ..types import RegularizerMode


class Regularizer:
    type = RegularizerMode.REG_MODE_NONE
    _lambda = 0.0


class L1(Regularizer):
    def __init__(self, l1=0.01):
        self.type = RegularizerMode.REG_MODE_L1
        self._lambda = float(l1)


class L2(Regularizer):
    def __init__(self, l2=0.01):
        self.type = RegularizerMode.REG_MODE_L2
        self._lambda = float(l2)
