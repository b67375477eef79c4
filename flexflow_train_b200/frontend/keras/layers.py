"""Keras-style layers that build onto an ``FFModel`` (bindings/python/old/flexflow/keras/layers/*.py).

A layer is called on symbolic ``KTensor`` objects (functional API) or stacked in ``Sequential``; ``Model`` later
replays the recorded calls against an ``FFModel``.  Shapes exclude the batch dimension, as in Keras; 4-D data is
channels-first (N, C, H, W), which is what the legacy frontend used too.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

from ..types import ActiMode, AggrMode, DataType, PoolType

_ACTS = {None: ActiMode.AC_MODE_NONE, "linear": ActiMode.AC_MODE_NONE, "relu": ActiMode.AC_MODE_RELU,
         "sigmoid": ActiMode.AC_MODE_SIGMOID, "tanh": ActiMode.AC_MODE_TANH, "gelu": ActiMode.AC_MODE_GELU}


class KTensor:
    """Symbolic output of a layer call."""

    def __init__(self, layer: Optional["Layer"], inputs: Sequence["KTensor"], shape=None, dtype="float32", index=0):
        self.layer, self.inputs, self.shape, self.dtype, self.index = layer, list(inputs), shape, dtype, index
        self.ff = None  # bound frontend Tensor while a Model is being built


class Layer:
    _count = {}

    def __init__(self, name=None, **kw):
        base = type(self).__name__.lower()
        n = Layer._count.get(base, 0)
        Layer._count[base] = n + 1
        self.name = name or (f"{base}_{n}" if n else base)
        self.input_shape = kw.get("input_shape")

    def __call__(self, x):
        xs = list(x) if isinstance(x, (list, tuple)) else [x]
        return KTensor(self, xs)

    def build(self, ff, inputs):
        raise NotImplementedError


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _init(v):
    """A Keras initializer (object or name) or a layer-API initializer -> what the layer API takes."""
    if v is None:
        return None
    from . import initializers
    if isinstance(v, str):
        v = initializers.get(v)
    return v.ff() if isinstance(v, initializers.Initializer) else v


def _padding(p, k):
    if p == "valid":
        return (0, 0)
    if p == "same":
        return (k[0] // 2, k[1] // 2)
    return _pair(p)


class InputLayer(Layer):
    def __init__(self, shape, dtype="float32", name=None):
        super().__init__(name)
        self.shape, self.dtype = tuple(shape), dtype


def Input(shape, dtype="float32", name=None):
    l = InputLayer(shape, dtype, name)
    return KTensor(l, [], shape=tuple(shape), dtype=dtype)


class Dense(Layer):
    def __init__(self, units, activation=None, use_bias=True, kernel_initializer=None, bias_initializer=None, name=None, **kw):
        super().__init__(name, **kw)
        self.units, self.activation, self.use_bias = units, activation, use_bias
        self.kernel_initializer, self.bias_initializer = _init(kernel_initializer), _init(bias_initializer)
        self.kernel_regularizer = kw.get("kernel_regularizer")     # recorded; see keras/regularizers.py

    def build(self, ff, xs):
        act = self.activation
        if act == "softmax":
            return ff.softmax(ff.dense(xs[0], self.units, ActiMode.AC_MODE_NONE, self.use_bias, kernel_initializer=self.kernel_initializer,
                                       bias_initializer=self.bias_initializer, name=self.name), name=self.name + "_softmax")
        return ff.dense(xs[0], self.units, _ACTS[act], self.use_bias, kernel_initializer=self.kernel_initializer,
                        bias_initializer=self.bias_initializer, name=self.name)


class Conv2D(Layer):
    def __init__(self, filters, kernel_size, strides=(1, 1), padding="valid", activation=None, groups=1, use_bias=True,
                 kernel_initializer=None, bias_initializer=None, name=None, **kw):
        super().__init__(name, **kw)
        self.filters, self.kernel, self.strides, self.padding = filters, _pair(kernel_size), _pair(strides), padding
        self.activation, self.groups, self.use_bias = activation, groups, use_bias
        self.kernel_initializer, self.bias_initializer = _init(kernel_initializer), _init(bias_initializer)

    def build(self, ff, xs):
        p = _padding(self.padding, self.kernel)
        return ff.conv2d(xs[0], self.filters, self.kernel[0], self.kernel[1], self.strides[0], self.strides[1], p[0], p[1],
                         _ACTS[self.activation], self.groups, self.use_bias, kernel_initializer=self.kernel_initializer,
                         bias_initializer=self.bias_initializer, name=self.name)


class _Pool2D(Layer):
    kind = PoolType.POOL_MAX

    def __init__(self, pool_size=(2, 2), strides=None, padding="valid", name=None, **kw):
        super().__init__(name, **kw)
        self.pool, self.padding = _pair(pool_size), padding
        self.strides = _pair(strides) if strides is not None else self.pool

    def build(self, ff, xs):
        p = _padding(self.padding, self.pool)
        return ff.pool2d(xs[0], self.pool[0], self.pool[1], self.strides[0], self.strides[1], p[0], p[1], self.kind, name=self.name)


class MaxPooling2D(_Pool2D):
    kind = PoolType.POOL_MAX


class AveragePooling2D(_Pool2D):
    kind = PoolType.POOL_AVG


class Flatten(Layer):
    def build(self, ff, xs):
        return ff.flat(xs[0], name=self.name)


class Dropout(Layer):
    def __init__(self, rate, seed=0, name=None, **kw):
        super().__init__(name, **kw)
        self.rate, self.seed = rate, seed

    def build(self, ff, xs):
        return ff.dropout(xs[0], self.rate, self.seed, name=self.name)


class Activation(Layer):
    def __init__(self, activation, name=None, **kw):
        super().__init__(name, **kw)
        self.activation = activation

    def build(self, ff, xs):
        if self.activation == "softmax":
            return ff.softmax(xs[0], name=self.name)
        if self.activation in (None, "linear"):
            return ff.identity(xs[0], name=self.name)
        return getattr(ff, self.activation)(xs[0], name=self.name)


class BatchNormalization(Layer):
    def build(self, ff, xs):
        return ff.batch_norm(xs[0], relu=False, name=self.name)


class LayerNormalization(Layer):
    def __init__(self, axis=-1, epsilon=1e-3, name=None, **kw):
        super().__init__(name, **kw)
        self.axis, self.eps = axis, epsilon

    def build(self, ff, xs):
        axes = [self.axis] if isinstance(self.axis, int) else list(self.axis)
        return ff.layer_norm(xs[0], axes, True, self.eps, name=self.name)


class Embedding(Layer):
    def __init__(self, input_dim, output_dim, embeddings_initializer=None, name=None, **kw):
        super().__init__(name, **kw)
        self.input_dim, self.output_dim, self.init = input_dim, output_dim, embeddings_initializer

    def build(self, ff, xs):
        return ff.embedding(xs[0], self.input_dim, self.output_dim, AggrMode.AGGR_MODE_SUM, kernel_initializer=self.init, name=self.name)


class Reshape(Layer):
    def __init__(self, target_shape, name=None, **kw):
        super().__init__(name, **kw)
        self.target = tuple(target_shape)

    def build(self, ff, xs):
        return ff.reshape(xs[0], [xs[0].dims[0]] + list(self.target), name=self.name)


class Permute(Layer):
    def __init__(self, dims, name=None, **kw):
        super().__init__(name, **kw)
        self.dims = tuple(dims)

    def build(self, ff, xs):
        return ff.transpose(xs[0], [0] + [int(d) for d in self.dims], name=self.name)


class Concatenate(Layer):
    def __init__(self, axis=1, name=None, **kw):
        super().__init__(name, **kw)
        self.axis = axis

    def build(self, ff, xs):
        return ff.concat(xs, self.axis, name=self.name)


class _Merge(Layer):
    op = "add"

    def build(self, ff, xs):
        out = xs[0]
        for other in xs[1:]:
            out = getattr(ff, self.op)(out, other, name=self.name)
        return out


class Add(_Merge):
    op = "add"


class Subtract(_Merge):
    op = "subtract"


class Multiply(_Merge):
    op = "multiply"


class Maximum(_Merge):
    op = "max"


class Minimum(_Merge):
    op = "min"


def concatenate(tensors, axis=1):
    return Concatenate(axis)(tensors)


def add(tensors):
    return Add()(tensors)


def subtract(tensors):
    return Subtract()(tensors)


def multiply(tensors):
    return Multiply()(tensors)
