"""Keras-style initializers (bindings/python/old/flexflow/keras/initializers.py): thin classes that produce the layer API's
initializer objects; pass them as ``kernel_initializer`` / ``bias_initializer``."""
from ..ffmodel import GlorotUniformInitializer, NormInitializer, UniformInitializer, ZeroInitializer


class Initializer:
    def ff(self):
        """The initializer object of the layer API, or None for the layer's default."""
        return None


class DefaultInitializer(Initializer):
    pass


class Zeros(Initializer):
    def ff(self):
        return ZeroInitializer()


class GlorotUniform(Initializer):
    def __init__(self, seed=0):
        self.seed = int(seed or 0)

    def ff(self):
        return GlorotUniformInitializer(self.seed)


class RandomUniform(Initializer):
    def __init__(self, minval=-0.05, maxval=0.05, seed=0):
        self.minval, self.maxval, self.seed = float(minval), float(maxval), int(seed or 0)

    def ff(self):
        return UniformInitializer(self.seed, self.minval, self.maxval)


class RandomNormal(Initializer):
    def __init__(self, mean=0.0, stddev=0.05, seed=0):
        self.mean, self.stddev, self.seed = float(mean), float(stddev), int(seed or 0)

    def ff(self):
        return NormInitializer(self.seed, self.mean, self.stddev)


def get(identifier):
    """An initializer from a name, an instance or None."""
    if identifier is None or isinstance(identifier, Initializer):
        return identifier
    table = {"zeros": Zeros, "glorot_uniform": GlorotUniform, "random_uniform": RandomUniform, "random_normal": RandomNormal}
    try:
        return table[str(identifier).lower()]()
    except KeyError:
        raise ValueError(f"unknown initializer {identifier!r}") from None
