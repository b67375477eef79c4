"""Keras backend functions on symbolic tensors (bindings/python/old/flexflow/keras/backend/backend_functions.py, internal.py):
each is a small layer, so that it can be used inside a functional model like any other layer."""
from .layers import Layer


class _Fn(Layer):
    def __init__(self, fn, name=None, **params):
        super().__init__(name)
        self.fn, self.params = fn, params

    def build(self, ff, xs):
        return self.fn(ff, xs, self.name, **self.params)


def _unary(method):
    def make(x, *args):
        return _Fn(lambda ff, xs, name, a=args: getattr(ff, method)(xs[0], *a, name=name))(x)
    return make


sin = _unary("sin")
cos = _unary("cos")
exp = _unary("exp")
rsqrt = _unary("rsqrt")


def pow(x, a):   # noqa: A001  (the Keras name)
    return _Fn(lambda ff, xs, name: ff.pow(xs[0], float(a), name=name))(x)


def sum(x, axis=None, keepdims=False):   # noqa: A001
    """Sum over `axis` (an int or a list; axes count the batch dim as 0, as in Keras)."""
    if axis is None:
        raise ValueError("backend.sum needs the axis to reduce")
    axes = [axis] if isinstance(axis, int) else list(axis)
    return _Fn(lambda ff, xs, name: ff.reduce_sum(xs[0], axes, keepdims, name=name))(x)


def batch_dot(x, y):
    """Batched matrix product of two 3-d tensors: [b, n, m] x [b, m, p] -> [b, n, p]."""
    return _Fn(lambda ff, xs, name: ff.batch_matmul(xs[0], xs[1], name=name))([x, y])


def gather(x, indices, axis):
    return _Fn(lambda ff, xs, name: ff.gather(xs[0], xs[1], int(axis), name=name))([x, indices])
