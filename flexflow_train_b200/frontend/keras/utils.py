"""Keras utilities (bindings/python/old/flexflow/keras/utils/np_utils.py)."""
import numpy as np


def to_categorical(y, num_classes=None, dtype="float32"):
    """Class vector (integers 0..num_classes-1, any shape, a trailing 1 is dropped) -> one-hot matrix."""
    y = np.asarray(y, dtype="int64")
    shape = y.shape
    if shape and shape[-1] == 1 and len(shape) > 1:
        shape = shape[:-1]
    y = y.ravel()
    if y.size and y.min() < 0:
        raise ValueError("to_categorical: negative class index")
    n = int(num_classes) if num_classes else (int(y.max()) + 1 if y.size else 0)
    if y.size and y.max() >= n:
        raise ValueError(f"to_categorical: class {int(y.max())} with num_classes={n}")
    out = np.zeros((y.shape[0], n), dtype=dtype)
    out[np.arange(y.shape[0]), y] = 1
    return out.reshape(shape + (n,))


def normalize(x, axis=-1, order=2):
    """x / ||x|| along `axis` (zero vectors stay zero)."""
    x = np.asarray(x, dtype="float64")
    norm = np.atleast_1d(np.linalg.norm(x, order, axis))
    norm[norm == 0] = 1
    return x / np.expand_dims(norm, axis)
