"""Keras-style optimizers (bindings/python/old/flexflow/keras/optimizers.py)."""
from ..ffmodel import AdamOptimizer, SGDOptimizer


class SGD(SGDOptimizer):
    def __init__(self, learning_rate=0.01, momentum=0.0, nesterov=False, weight_decay=0.0, lr=None):
        super().__init__(None, lr if lr is not None else learning_rate, momentum, nesterov, weight_decay)


class Adam(AdamOptimizer):
    def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.999, epsilon=1e-8, weight_decay=0.0, lr=None):
        super().__init__(None, lr if lr is not None else learning_rate, beta_1, beta_2, weight_decay, epsilon)


def get(identifier):
    if isinstance(identifier, (SGDOptimizer, AdamOptimizer)):
        return identifier
    return {"sgd": SGD, "adam": Adam}[str(identifier).lower()]()
